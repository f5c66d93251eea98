"""Typed configuration of the Dobelix decoder, read from its config.json.

A Dobelix model is a list of layers, each with one of two mixers (``lightning``: linear
attention with a decay per head; ``attention``: grouped-query attention with sigmoid weights
inside chunks of positions) and, optionally, a dense gated feed-forward.  Every size and every
constant that differs between models comes from config.json; nothing here has a default that a
model could silently fall back on.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError


def _get(d: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing key {key!r} in {where}")
    return d[key]


def _int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _get(d, key, where)
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _num(d: Mapping[str, Any], key: str, where: str) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class ChunkAttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class DobelixLayer:
    type: str
    mixer: Any
    mlp: Optional[DenseMlp]


@dataclass(frozen=True)
class DobelixConfig:
    vocab: int
    width: int
    layers: Tuple[DobelixLayer, ...]
    eps: float
    taps: int
    embedding_scale: float
    logit_scale: float
    max_positions: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DobelixConfig":
        layers = _get(d, "layers", "config")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            m = _get(entry, "mixer", where)
            mw = where + ".mixer"
            if kind == "lightning":
                heads = _int(m, "heads", mw)
                decay = _get(m, "decay", mw)
                if not isinstance(decay, (list, tuple)) or len(decay) != heads:
                    raise ConfigError(f"config.json: {mw}.decay must list one number per head ({heads})")
                mixer = LightningMixer(heads, _int(m, "dim", mw), _int(m, "vdim", mw), tuple(float(x) for x in decay))
            elif kind == "attention":
                heads, kv = _int(m, "heads", mw), _int(m, "kv_heads", mw)
                if heads % kv:
                    raise ConfigError(f"config.json: {mw}.heads {heads} must be a multiple of kv_heads {kv}")
                dim, vdim = _int(m, "dim", mw), _int(m, "vdim", mw)
                if vdim != dim:
                    raise ConfigError(f"config.json: {mw}: the values are the keys, so vdim {vdim} must equal dim {dim}")
                rot = _get(m, "rot", mw)
                rot_dims = _int(rot, "dims", mw + ".rot")
                if rot_dims % 2 or rot_dims > dim:
                    raise ConfigError(f"config.json: {mw}.rot.dims {rot_dims} must be even and at most dim {dim}")
                mixer = ChunkAttentionMixer(heads, kv, dim, vdim, _num(m, "scale", mw),
                                            _int(_get(m, "mask", mw), "size", mw + ".mask"), rot_dims,
                                            _num(rot, "base", mw + ".rot"))
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  "(known: lightning, attention)")
            mlp = entry.get("mlp") if isinstance(entry, Mapping) else None
            if mlp is not None:
                mk = _get(mlp, "kind", where + ".mlp")
                if mk != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mk!r} is not a feed-forward of this design (known: dense)")
                mlp = DenseMlp(_int(mlp, "ff", where + ".mlp"))
            out.append(DobelixLayer(kind, mixer, mlp))
        max_positions = d.get("max_positions", d.get("max_position_embeddings", 1 << 20))
        return cls(vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"), layers=tuple(out),
                   eps=_num(_get(d, "norm", "config"), "eps", "norm"),
                   taps=_int(_get(d, "canon", "config"), "taps", "canon"),
                   embedding_scale=_num(_get(d, "embedding", "config"), "scale", "embedding"),
                   logit_scale=_num(d, "logit_scale", "config"), max_positions=int(max_positions))
