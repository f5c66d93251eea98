"""Attention through low-rank latents with one rotated key part shared by all heads.

With x the mixer's input, per token::

    c_q = N(W_dq x)                 query latent, RMS norm with a weight
    q_h = W_uq,h c_q                per head [plain part of head_dim | part of rope_dim to rotate]
    [c | r] = W_dkv x               c: key/value latent (then c = N(c)), r: rope_dim numbers, rotated
    k_h = [W_uk,h c | rot(r)]       v_h = W_uv,h c

Only [c | rot(r)] is cached: one vector of kv_rank + rope_dim numbers per token, for all heads.  The scores are
taken against it directly, q_h.k_h = (W_uk,h^T q_h,plain).c + rot(q_h,rot).rot(r), and the heads' values are
expanded after the weighted sum, o_h = W_uv,h (sum_j p_j c_j): attention with a single cached "head" whose keys
have kv_rank + rope_dim dimensions and whose values are the first kv_rank of them.  Softmax over a causal
(optionally sliding) window; ``gate="head"`` multiplies head h's output by sigmoid(W_g x)_h.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..cache.needs import PagedKV
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Mixer, build_part, register_part
from .gated_attention import pad8


class LatentAttention(Mixer):
    """spec: ``width``, ``heads``, ``head_dim`` (plain query/key dimensions), ``rope_dim`` (rotated ones), ``value_dim``,
    ``q_rank``, ``kv_rank``, ``position`` (a PartSpec over ``rope_dim``), ``scale``, ``window``, ``eps`` (of the latents'
    norms), ``gate``."""
    can_overwrite = True

    @property
    def graph_safe(self) -> bool:
        return bool(self.position.graph_safe)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        h, d, r, v = spec.heads, spec.head_dim, spec.rope_dim, spec.value_dim
        needs = {"dq": TensorNeed((spec.q_rank, spec.width)), "dq_norm": TensorNeed((spec.q_rank,), role="scale"),
                 "uq": TensorNeed((h * (d + r), spec.q_rank)),
                 "dkv": TensorNeed((spec.kv_rank + r, spec.width)), "dkv_norm": TensorNeed((spec.kv_rank,), role="scale"),
                 "uk": TensorNeed((h * d, spec.kv_rank)), "uv": TensorNeed((h * v, spec.kv_rank)),
                 "o": TensorNeed((spec.width, h * v))}
        if spec.get("gate") == "head":
            needs["g"] = TensorNeed((h, spec.width))
        return needs

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.head_dim, self.rope_dim = int(spec.heads), int(spec.head_dim), int(spec.rope_dim)
        self.value_dim, self.q_rank, self.kv_rank = int(spec.value_dim), int(spec.q_rank), int(spec.kv_rank)
        if spec.get("gate") not in (None, "head"):
            raise ValueError(f"gate must be 'head' or None, got {spec.get('gate')!r}")
        self.window = spec.get("window")
        self.scale, self.eps = float(spec.scale), float(spec.eps)
        self.position = build_part("position", spec.position, {}, rt)
        if self.position.rope_dim != self.rope_dim or self.position.interleaved:
            raise ValueError("the shared key part is rotated as a whole, dimension i with i + rope_dim/2")
        self.cached_dim = self.kv_rank + self.rope_dim
        # one fused projection of the input: rows [query latent | key/value latent | tail to rotate | gate (if gated)]
        rows = [tensors["dq"], tensors["dkv"]]
        self.g_at = None
        if "g" in tensors:
            self.g_at = self.q_rank + self.cached_dim
            rows.append(tensors["g"])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.in_cols = self.w_in.shape[0]
        self.q_norm, self.kv_norm = tensors["dq_norm"], tensors["dkv_norm"]
        self.w_uq = tensors["uq"]
        h, d, v, rank = self.heads, self.head_dim, self.value_dim, self.kv_rank
        self.w_fold = tensors["uk"].reshape(h, d, rank).transpose(1, 2).contiguous()      # [h, rank, d]: W_uk,h^T
        self.w_uv = tensors["uv"].reshape(h, v, rank).contiguous()
        self.w_o = tensors["o"]

    def cache_need(self) -> PagedKV:
        return PagedKV(1, self.cached_dim, self.window, None, 0)

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: Any, cache: Any, writes_cache: bool,
                accumulate: bool = True) -> None:
        n, rt = step.n, self.rt
        x = x if isinstance(x, torch.Tensor) else x.tensor()
        h, d, r, v, rank = self.heads, self.head_dim, self.rope_dim, self.value_dim, self.kv_rank
        cs = self.position.table(step)
        proj = rt.scratch("lattn_proj", (rt.max_tokens, pad8(self.in_cols)))[:n, :self.in_cols]
        ops.tag("qkv")
        ops.linear(x, self.w_in, proj)
        cq = rt.scratch("lattn_cq", (rt.max_tokens, pad8(self.q_rank)))[:n, :self.q_rank]
        ops.tag("rope")
        ops.latent_norm_rope_cache(proj, 0, self.q_rank, self.q_rank, rank, r, self.q_norm, self.kv_norm, self.eps, cs,
                                   step.positions, step.slot_of_token, cq, cache.k if writes_cache else None,
                                   cache.block_table, cache.page_size)
        qh = rt.scratch("lattn_q", (rt.max_tokens, pad8(h * (d + r))))[:n, :h * (d + r)]
        ops.tag("qkv")
        ops.linear(cq, self.w_uq, qh)
        # the query against the cached vector: [W_uk,h^T q_plain | rot(q_rot)] per head
        qf = rt.scratch("lattn_qfold", (rt.max_tokens, pad8(h * self.cached_dim)))[:n, :h * self.cached_dim]
        ops.tag("fold")
        ops.head_linear(qh, 0, d + r, self.w_fold, qf, 0, self.cached_dim)
        ops.tag("rope")
        ops.rope_norm_cache(qh, cs, r, None, step.positions, step.slot_of_token, cache.block_table, cache.page_size,
                            q=(h, d, d + r, r, 0, qf, rank, self.cached_dim))
        ol = rt.scratch("lattn_latent_out", (rt.max_tokens, pad8(h * rank)))[:n, :h * rank]
        ops.tag("attention")
        ops.latent_attention(qf, cache.k, cache.block_table, cache.page_size, step, ol, h, self.cached_dim, rank,
                             self.scale, int(self.window or 0))
        att = rt.scratch("lattn_out", (rt.max_tokens, pad8(h * v)))[:n, :h * v]
        gate = proj[:, self.g_at:self.g_at + h] if self.g_at is not None else None
        ops.tag("expand")
        ops.head_linear(ol, 0, rank, self.w_uv, att, 0, v, gate)
        ops.tag("o")
        ops.linear(att, self.w_o, out, accumulate=accumulate)


register_part("mixer", "latent_attention", LatentAttention)
