"""Grouped-query attention with unnormalised sigmoid weights over the paged cache.

Differences from :class:`~hfee_b200.parts.attention.PagedAttention`, each a parameter:

* the weight of a visible key is ``sigmoid(q.k * scale * temp[h] + bias[h])``; nothing is
  normalised over the keys (``head_temperature`` / ``head_bias`` say whether the per-head
  numbers exist);
* ``chunk``: a query at position i sees key j <= i only if both lie in the same block of
  ``chunk`` positions counted from position 0 of the request (None: plain causal);
* ``qk_norm_eps``: queries and keys are RMS-normed over the whole projection (all heads at
  once) before the rotation (None: no norm);
* ``values``: ``"keys"`` takes the key projection, as it came out of W_k, for the values
  (there is no W_v); ``"projected"`` has a W_v;
* ``gate``: the heads' outputs are multiplied by ``sigmoid(W_g h)`` before the output projection.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..cache.needs import PagedKV
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Mixer, build_part, register_part


class SigmoidAttention(Mixer):
    """spec: ``width``, ``heads``, ``kv_heads``, ``head_dim``, ``position`` (a PartSpec), ``scale``,
    ``chunk``, ``window``, ``qk_norm_eps``, ``values``, ``gate``, ``head_temperature``, ``head_bias``."""
    can_overwrite = True

    @property
    def graph_safe(self) -> bool:
        return bool(self.position.graph_safe)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        q, kv = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim
        needs = {"q": TensorNeed((q, spec.width)), "k": TensorNeed((kv, spec.width)), "o": TensorNeed((spec.width, q))}
        if spec.get("values", "projected") == "projected":
            needs["v"] = TensorNeed((kv, spec.width))
        if spec.get("qk_norm_eps") is not None:
            needs["q_norm"] = TensorNeed((q,), role="scale")
            needs["k_norm"] = TensorNeed((kv,), role="scale")
        if spec.get("gate", False):
            needs["g"] = TensorNeed((q, spec.width))
        if spec.get("head_temperature", False):
            needs["temp"] = TensorNeed((spec.heads,), role="scale")
        if spec.get("head_bias", False):
            needs["bias"] = TensorNeed((spec.heads,), role="vector")
        return needs

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.kv_heads, self.head_dim = int(spec.heads), int(spec.kv_heads), int(spec.head_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} must be a multiple of kv_heads {self.kv_heads}")
        self.values = spec.get("values", "projected")
        if self.values not in ("projected", "keys"):
            raise ValueError(f"values must be 'projected' or 'keys', got {self.values!r}")
        self.chunk, self.window = spec.get("chunk"), spec.get("window")
        if self.chunk is not None and int(self.chunk) < 1:
            raise ValueError(f"chunk must be positive, got {self.chunk}")
        self.scale = float(spec.scale)
        self.eps = spec.get("qk_norm_eps")
        self.position = build_part("position", spec.position, {}, rt)
        if self.position.rope_dim and self.position.interleaved:
            raise ValueError("this attention rotates dimension i with i + rope_dim/2 only")
        self.q_cols, self.kv_cols = self.heads * self.head_dim, self.kv_heads * self.head_dim
        # one fused projection: rows [q | k | v (if projected) | g (if gated)]
        rows = [tensors["q"], tensors["k"]]
        self.v_at = self.g_at = None
        at = self.q_cols + self.kv_cols
        if self.values == "projected":
            rows.append(tensors["v"]); self.v_at = at; at += self.kv_cols
        if "g" in tensors:
            rows.append(tensors["g"]); self.g_at = at; at += self.q_cols
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.in_cols = at
        self.w_o = tensors["o"]
        self.q_norm, self.k_norm = tensors.get("q_norm"), tensors.get("k_norm")
        self.temp, self.bias = tensors.get("temp"), tensors.get("bias")

    def cache_need(self) -> PagedKV:
        return PagedKV(self.kv_heads, self.head_dim, self.window, int(self.chunk) if self.chunk is not None else None)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool,
                accumulate: bool = True) -> None:
        n, rt = step.n, self.rt
        h = h if isinstance(h, torch.Tensor) else h.tensor()
        cs = self.position.table(step)
        w = self.w_in
        if not writes_cache and self.g_at is None:
            w = self.w_in[:self.q_cols]             # a run over another run's cache projects queries only
        proj = rt.scratch("sigattn_proj", (rt.max_tokens, self.in_cols))[:n, :w.shape[0]]
        ops.tag("qkv")
        ops.linear(h, w, proj)
        q = rt.scratch("attn_q", (rt.max_tokens, self.q_cols))[:n]
        k_pool, v_pool = (cache.k, cache.v) if writes_cache else (None, None)
        ops.tag("rope")
        ops.qk_norm_rope_cache(proj, self.q_norm, self.k_norm, float(self.eps or 0.0), cs, self.position.rope_dim,
                               step.positions, step.slot_of_token, q, k_pool, v_pool, cache.block_table,
                               cache.page_size, self.heads, self.kv_heads, self.head_dim,
                               v_offset=-1 if self.values == "keys" else self.v_at)
        att = rt.scratch("attn_out", (rt.max_tokens, self.q_cols))[:n]
        gate = proj[:, self.g_at:self.g_at + self.q_cols] if self.g_at is not None else None
        ops.tag("attention")
        ops.sigmoid_attention(q, cache.k, cache.v, cache.block_table, cache.page_size, step, att, self.heads,
                              self.kv_heads, self.head_dim, self.scale, int(self.window or 0), int(self.chunk or 0),
                              self.temp, self.bias, gate)
        ops.tag("o")
        ops.linear(att, self.w_o, residual, accumulate=accumulate)


register_part("mixer", "sigmoid_attention", SigmoidAttention)
