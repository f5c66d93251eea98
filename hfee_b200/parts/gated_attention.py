"""Grouped-query softmax attention with independent key and value sizes, a partial rotation, queries
and keys brought to unit root mean square, and a gate on the heads' outputs.

Differences from :class:`~hfee_b200.parts.attention.PagedAttention`, each a parameter:

* ``value_dim``: a value's size need not be the key's (the cache keeps values in a pool of their own shape);
* the rotation covers the first ``rope_dim`` dimensions of a head and pairs dimension i with i + rope_dim/2;
* ``qk_unit_norm_eps``: after the rotation every query and key head is divided by sqrt(mean(x^2) + eps),
  without a weight (None: no norm);
* ``gate``: ``"head"`` multiplies head h's output by sigmoid(W_g x)_h, one number per head and token, before the
  output projection (None: no gate);
* ``window``: a query sees itself and the ``window - 1`` positions before it (None: all earlier positions).
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..cache.needs import PagedKV
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Mixer, build_part, register_part


def pad8(n: int) -> int:
    """Row strides of activation buffers are multiples of 8 elements, so that every row starts on 16 bytes."""
    return -(-n // 8) * 8


class GatedAttention(Mixer):
    """spec: ``width``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``position`` (a PartSpec), ``scale``,
    ``window``, ``qk_unit_norm_eps``, ``gate``."""
    can_overwrite = True

    @property
    def graph_safe(self) -> bool:
        return bool(self.position.graph_safe)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        q, k, v = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim, spec.kv_heads * spec.value_dim
        needs = {"q": TensorNeed((q, spec.width)), "k": TensorNeed((k, spec.width)), "v": TensorNeed((v, spec.width)),
                 "o": TensorNeed((spec.width, spec.heads * spec.value_dim))}
        if spec.get("gate") == "head":
            needs["g"] = TensorNeed((spec.heads, spec.width))
        return needs

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.kv_heads = int(spec.heads), int(spec.kv_heads)
        self.head_dim, self.value_dim = int(spec.head_dim), int(spec.value_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} must be a multiple of kv_heads {self.kv_heads}")
        if spec.get("gate") not in (None, "head"):
            raise ValueError(f"gate must be 'head' or None, got {spec.get('gate')!r}")
        self.window = spec.get("window")
        self.scale = float(spec.scale)
        self.eps = spec.get("qk_unit_norm_eps")
        self.position = build_part("position", spec.position, {}, rt)
        if self.position.rope_dim and self.position.interleaved:
            raise ValueError("this attention rotates dimension i with i + rope_dim/2 only")
        self.q_cols, self.k_cols = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.v_cols, self.o_cols = self.kv_heads * self.value_dim, self.heads * self.value_dim
        # one fused projection: rows [q | k | v | g (if gated)]
        rows = [tensors["q"], tensors["k"], tensors["v"]]
        self.g_at = None
        if "g" in tensors:
            self.g_at = self.q_cols + self.k_cols + self.v_cols
            rows.append(tensors["g"])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.in_cols = self.w_in.shape[0]
        self.w_o = tensors["o"]
        self.split_scratch = None
        if self.head_dim == self.value_dim:        # the tensor-core kernels' partial results of split decode steps
            self.split_scratch = rt.scratch("attn_partials", (rt.max_requests * self.heads * ops.MAX_SPLITS *
                                                              (self.head_dim + 2),), torch.float32)

    def cache_need(self) -> PagedKV:
        return PagedKV(self.kv_heads, self.head_dim, self.window, None, self.value_dim)

    def forward(self, h: torch.Tensor, out: torch.Tensor, step: Any, cache: Any, writes_cache: bool,
                accumulate: bool = True) -> None:
        n, rt = step.n, self.rt
        h = h if isinstance(h, torch.Tensor) else h.tensor()
        cs = self.position.table(step)
        w = self.w_in
        if not writes_cache and self.g_at is None:
            w = self.w_in[:self.q_cols]             # a run over another run's cache projects queries only
        proj = rt.scratch("gattn_proj", (rt.max_tokens, pad8(self.in_cols)))[:n, :w.shape[0]]
        ops.tag("qkv")
        ops.linear(h, w, proj)
        q = rt.scratch("attn_q", (rt.max_tokens, self.q_cols))[:n]
        d = self.head_dim
        ops.tag("rope")
        ops.rope_norm_cache(proj, cs, self.position.rope_dim, self.eps, step.positions, step.slot_of_token,
                            cache.block_table, cache.page_size, q=(self.heads, 0, d, d, 0, q, 0, d),
                            k=(self.kv_heads, self.q_cols, d, d, 0, cache.k, 0) if writes_cache else None,
                            v=(self.q_cols + self.k_cols, self.value_dim, self.value_dim, cache.v) if writes_cache else None)
        att = rt.scratch("gattn_out", (rt.max_tokens, pad8(self.o_cols)))[:n, :self.o_cols]
        gate = proj[:, self.g_at:self.g_at + self.heads] if self.g_at is not None else None
        ops.tag("attention")
        if ops.softmax_attention_on_tensor_cores(q, att, self.heads, self.kv_heads, self.head_dim, self.value_dim,
                                                 cache.page_size, step):
            ops.paged_attention(q, cache.k, cache.v, cache.block_table, cache.page_size, step.positions,
                                step.slot_of_token, att, self.heads, self.kv_heads, self.head_dim, self.scale,
                                int(self.window or 0), step=step, scratch=self.split_scratch)
            if gate is not None:
                ops.head_gate(att, gate, self.heads, self.value_dim)
        else:
            ops.attention_simt_general(q, cache.k, cache.v, cache.block_table, cache.page_size, step.positions,
                                       step.slot_of_token, att, self.heads, self.kv_heads, self.head_dim, self.value_dim,
                                       self.scale, int(self.window or 0), 0, gate,
                                       ops.GATE_PER_HEAD if gate is not None else ops.GATE_NONE)
        ops.tag("o")
        ops.linear(att, self.w_o, out, accumulate=accumulate)


register_part("mixer", "gated_attention", GatedAttention)
