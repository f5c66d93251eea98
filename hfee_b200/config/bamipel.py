"""Typed configuration of the Bamipel decoder, read from its config.json.

A Bamipel model is a list of layers, each with one of three mixers and, optionally, a dense
feed-forward; a layer may name another layer whose tensors it uses (``weights_of``) and then keeps
only a cache or state of its own.  The mixers: ``attention`` (grouped-query softmax attention with a
partial rotation, unit-RMS queries and keys and one gate per head), ``latent_attention`` (queries
and keys/values through low-rank latents, one rotated key part for all heads, a sliding window) and
``delta`` (the gated delta rule behind short convolutions).  Every size and every constant that
differs between models comes from config.json; nothing here has a default that a model could
silently fall back on.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .dobelix import DenseMlp, _get, _int, _num
from .llama import ConfigError, RopeScaling


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: Optional[RopeScaling]


@dataclass(frozen=True)
class GatedAttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation
    window: Optional[int]


@dataclass(frozen=True)
class LatentAttentionMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Rotation
    window: Optional[int]


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int


@dataclass(frozen=True)
class BamipelLayer:
    type: str
    mixer: Any
    mlp: Optional[DenseMlp]
    weights_of: Optional[int]      # the layer whose tensors this one uses; None: its own


@dataclass(frozen=True)
class BamipelConfig:
    vocab: int
    width: int
    layers: Tuple[BamipelLayer, ...]
    eps: float
    max_positions: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BamipelConfig":
        layers = _get(d, "layers", "config")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            m = _get(entry, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                heads, kv = _int(m, "heads", mw), _int(m, "kv_heads", mw)
                if heads % kv:
                    raise ConfigError(f"config.json: {mw}.heads {heads} must be a multiple of kv_heads {kv}")
                dim = _int(m, "dim", mw)
                mixer = GatedAttentionMixer(heads, kv, dim, _int(m, "vdim", mw), _num(m, "scale", mw),
                                            _rotation(_get(m, "rot", mw), dim, mw + ".rot"), _window(m, mw))
            elif kind == "latent_attention":
                rot_dim = _int(m, "rot_dim", mw)
                rot = _rotation(_get(m, "rot", mw), rot_dim, mw + ".rot")
                if rot.dims != rot_dim:
                    raise ConfigError(f"config.json: {mw}.rot.dims {rot.dims} must equal rot_dim {rot_dim}: the whole "
                                      "shared key part is rotated")
                mixer = LatentAttentionMixer(_int(m, "heads", mw), _int(m, "dim", mw), rot_dim, _int(m, "vdim", mw),
                                             _int(m, "q_rank", mw), _int(m, "kv_rank", mw), _num(m, "scale", mw), rot,
                                             _window(m, mw))
            elif kind == "delta":
                heads, kv = _int(m, "heads", mw), _int(m, "kv_heads", mw)
                if heads % kv:
                    raise ConfigError(f"config.json: {mw}.heads {heads} must be a multiple of kv_heads {kv}")
                mixer = DeltaMixer(heads, kv, _int(m, "dim", mw), _int(m, "vdim", mw), _int(m, "conv", mw))
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  "(known: attention, latent_attention, delta)")
            mlp = entry.get("mlp") if isinstance(entry, Mapping) else None
            if mlp is not None:
                mk = _get(mlp, "kind", where + ".mlp")
                if mk != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mk!r} is not a feed-forward of this design (known: dense)")
                mlp = DenseMlp(_int(mlp, "ff", where + ".mlp"))
            source = entry.get("weights_of")
            if source is not None and (not isinstance(source, int) or isinstance(source, bool) or not 0 <= source < len(layers)):
                raise ConfigError(f"config.json: {where}.weights_of {source!r} is not a layer of this model")
            out.append(BamipelLayer(kind, mixer, mlp, source))
        for i, layer in enumerate(out):
            if layer.weights_of is None:
                continue
            src = out[layer.weights_of]
            if src.weights_of is not None:
                raise ConfigError(f"config.json: layers[{i}].weights_of names layer {layer.weights_of}, which has no tensors of its own")
            if (src.type, src.mixer, src.mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"config.json: layers[{i}] uses the tensors of layer {layer.weights_of} but describes another layer")
        max_positions = d.get("max_positions", d.get("max_position_embeddings", 1 << 20))
        return cls(vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"), layers=tuple(out),
                   eps=_num(_get(d, "norm", "config"), "eps", "norm"), max_positions=int(max_positions))


def _window(m: Mapping[str, Any], where: str) -> Optional[int]:
    mask = m.get("mask")
    return None if mask is None else _int(mask, "size", where + ".mask")


def _rotation(rot: Mapping[str, Any], head_dim: int, where: str) -> Rotation:
    dims = _int(rot, "dims", where)
    if dims % 2 or dims > head_dim:
        raise ConfigError(f"config.json: {where}.dims {dims} must be even and at most {head_dim}")
    sc = rot.get("scaling")
    scaling = None
    if sc is not None:
        sw = where + ".scaling"
        scaling = RopeScaling(factor=_num(sc, "factor", sw), low_freq_factor=_num(sc, "low", sw),
                              high_freq_factor=_num(sc, "high", sw),
                              original_max_position_embeddings=_int(sc, "original", sw))
    return Rotation(dims, _num(rot, "base", where), scaling)
