"""Fesorax: a decoder whose layers are listed one by one in ``config.json``.

Every layer is a post-norm block (x <- norm(alpha x + sublayer(x)), twice) whose mixer is either
softmax attention (unit-norm queries and keys, a learned bias by log-bucketed distance, a sliding
window that keeps the first tokens, a logistic gate per head, optionally on an earlier layer's keys
and values) or an mLSTM matrix memory, and whose feed-forward is a mixture of clamped gated experts
with a shared expert, or absent.  The keys of ``config.json``:

    architecture            "Fesorax"
    vocab, width            sizes of the embedding and the residual stream
    embedding.scale         factor on the embedding rows
    postln_alpha            alpha of the blocks
    norm.eps                eps of every norm (also of the unit norms inside the mixers)
    layers[i].type          "attention" | "mlstm"
    layers[i].mixer         attention: heads, kv_heads, dim, vdim, scale, bias_max, mask.size, mask.keep_first,
                            kv_from (optional: the layer whose keys and values are used);
                            mlstm: heads, dim, vdim, gate_cap
    layers[i].mlp           null, or kind "moe" with router.experts, router.top, expert.ff, expert.limit and
                            (optional) shared.ff, shared.limit
    max_positions           (optional) the longest sequence; the design itself has no limit

Sizes that the file's tensors fix (the number of distance buckets) are read from them when the
model is loaded from a folder; a configuration without a folder names them under ``bias_buckets``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, Optional

from .spec import (BiasAttentionSpec, ConfigError, MlstmSpec, ModelSpec, MoeSpec, PostNormBlockSpec, RmsNormSpec,
                   ScheduleEntry)

ARCHITECTURE = "Fesorax"
DEFAULT_MAX_POSITIONS = 1 << 20
DEFAULT_BIAS_BUCKETS = 64  # for configurations without a folder (random weights); a folder's tables say their own


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


@dataclass(frozen=True)
class FesoraxConfig:
    """The file as it was read (``text``: canonical JSON, so that the record is hashable and can be
    written back unchanged) plus the checked top-level numbers."""

    text: str
    vocab: int
    width: int
    n_layers: int
    max_positions: int

    @property
    def data(self) -> Dict[str, Any]:
        return json.loads(self.text)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FesoraxConfig":
        layers = _need(d, "layers", "the file")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        _num(_need(d, "embedding", "the file"), "scale", "embedding")
        if not _num(_need(d, "norm", "the file"), "eps", "norm") > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        _num(d, "postln_alpha", "the file")
        mp = d.get("max_positions") or DEFAULT_MAX_POSITIONS
        cfg = cls(text=json.dumps(d, sort_keys=True), vocab=_int(d, "vocab", "the file"), width=_int(d, "width", "the file"),
                  n_layers=len(layers), max_positions=int(mp))
        cfg.to_spec()  # every layer is checked by building its spec
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return self.data

    def with_max_positions(self, max_seq: int) -> "FesoraxConfig":
        if max_seq and 0 < max_seq < self.max_positions:
            d = self.data
            d["max_positions"] = int(max_seq)
            return FesoraxConfig.from_dict(d)
        return self

    # ---- translation into parts ------------------------------------------------------------
    def _mixer(self, i: int, layer: Dict[str, Any], eps: float, layers) -> Any:
        where = f"layers[{i}].mixer"
        m = _need(layer, "mixer", f"layers[{i}]")
        kind = _need(layer, "type", f"layers[{i}]")
        if kind == "mlstm":
            return MlstmSpec(width=self.width, n_heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
                             v_head_dim=_int(m, "vdim", where), gate_cap=_num(m, "gate_cap", where), norm_eps=eps)
        if kind != "attention":
            raise ConfigError(f"config.json: layers[{i}].type is 'attention' or 'mlstm', not {kind!r}")
        heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        dim = _int(m, "dim", where)
        if dim > 256 or _int(m, "vdim", where) > 256:
            raise ConfigError(f"config.json: {where}: dim={dim} and vdim={m['vdim']} must be at most 256")
        mask = m.get("mask") or {}
        src = m.get("kv_from")
        if src is not None:
            if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                raise ConfigError(f"config.json: {where}.kv_from={src!r} must name an earlier layer")
            other = layers[src]
            om = other.get("mixer") or {}
            if other.get("type") != "attention" or om.get("kv_from") is not None:
                raise ConfigError(f"config.json: {where}.kv_from={src}: that layer has no keys and values of its own")
            if (om.get("kv_heads"), om.get("dim"), om.get("vdim")) != (kv_heads, dim, m.get("vdim")):
                raise ConfigError(f"config.json: {where}.kv_from={src}: the two layers' kv_heads, dim and vdim differ")
        bias_max = _int(m, "bias_max", where)
        # without tables to read the number of rows from: the default, or fewer where the bias reaches less far
        buckets = int(m.get("bias_buckets") or max(2, min(DEFAULT_BIAS_BUCKETS, 2 * (bias_max - 1))))
        if bias_max <= buckets // 2:
            raise ConfigError(f"config.json: {where}.bias_max={bias_max} must exceed half the {buckets} distance buckets")
        return BiasAttentionSpec(
            width=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim, v_head_dim=_int(m, "vdim", where),
            scale=_num(m, "scale", where), window=int(mask.get("size") or 0), keep_first=int(mask.get("keep_first") or 0),
            unit_norm=True, norm_eps=eps, bias_buckets=buckets, bias_max_distance=bias_max, head_gate=True,
            own_kv=src is None)

    def _ffn(self, i: int, layer: Dict[str, Any]) -> Optional[MoeSpec]:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        where = f"layers[{i}].mlp"
        if mlp.get("kind", "moe") != "moe":
            raise ConfigError(f"config.json: {where}.kind is 'moe', not {mlp.get('kind')!r}")
        router, expert = _need(mlp, "router", where), _need(mlp, "expert", where)
        experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router.top={top} exceeds its {experts} experts")
        shared = mlp.get("shared")
        return MoeSpec(width=self.width, n_experts=experts, top=top, expert_ff=_int(expert, "ff", where + ".expert"),
                       expert_limit=_num(expert, "limit", where + ".expert"),
                       shared_ff=_int(shared, "ff", where + ".shared") if shared else 0,
                       shared_limit=_num(shared, "limit", where + ".shared") if shared else 0.0)

    def to_spec(self) -> ModelSpec:
        d = self.data
        eps, alpha = float(d["norm"]["eps"]), float(d["postln_alpha"])
        norm = RmsNormSpec(width=self.width, eps=eps)
        blocks, schedule = [], []
        for i, layer in enumerate(d["layers"]):
            mixer = self._mixer(i, layer, eps, d["layers"])
            ffn = self._ffn(i, layer)
            # without a feed-forward the second norm exists only if the file has its gain
            ffn_norm = norm if ffn is not None else RmsNormSpec(width=self.width, eps=eps, optional=True)
            blocks.append(PostNormBlockSpec(mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=ffn_norm, alpha=alpha))
            schedule.append(ScheduleEntry(block=i, cache_of=layer["mixer"].get("kv_from") if layer["type"] == "attention" else None))
        spec = ModelSpec(vocab_size=self.vocab, width=self.width, blocks=tuple(blocks), schedule=tuple(schedule),
                         final_norm=norm, max_positions=self.max_positions, embedding_scale=float(d["embedding"]["scale"]))
        spec.validate()
        return spec


def with_sizes_of(config: Dict[str, Any], shapes: Dict[str, Any]) -> Dict[str, Any]:
    """``config`` with the sizes that only the file's tensors fix filled in: the rows of each attention
    layer's distance-bias table."""
    out = json.loads(json.dumps(config))
    for i, layer in enumerate(out.get("layers") or []):
        shape = shapes.get(f"l{i}.mix.rel")
        if shape is not None and isinstance(layer.get("mixer"), dict):
            layer["mixer"]["bias_buckets"] = int(shape[0])
    return out


def tensor_name(path: str) -> str:
    """Checkpoint name of the parameter at ``path``: ``blocks.3.mixer.q`` is ``l3.mix.q``."""
    fixed = {"embedding.table": "embed", "final_norm.weight": "final.norm", "head.weight": "head"}
    if path in fixed:
        return fixed[path]
    parts = path.split(".")
    if parts[0] == "blocks" and len(parts) >= 4:
        i, role, rest = parts[1], parts[2], ".".join(parts[3:])
        if role == "mixer_norm" and rest == "weight":
            return f"l{i}.norm1"
        if role == "ffn_norm" and rest == "weight":
            return f"l{i}.norm2"
        if role == "mixer":
            return f"l{i}.mix.{rest}"
        if role == "ffn":
            return f"l{i}.mlp.{rest}"
    raise KeyError(f"the Fesorax architecture has no tensor for parameter '{path}'")
