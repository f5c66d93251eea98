"""The gated delta rule on a matrix state per head, behind short convolutions.

With x the mixer's input, per token t and head h (q, k of ``key_dim``, v of ``value_dim``)::

    q, k, v = silu(conv(W_q x)), silu(conv(W_k x)), silu(conv(W_v x))     causal convolutions over time per channel
    q = q / |q| * key_dim^-1/2,  k = k / |k|                               (|x| = sqrt(sum x^2 + 1e-6))
    beta = sigmoid(W_b x)_h      g = exp(-exp(A_log_h) * softplus((W_a x)_h + dt_bias_h))
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q

``qk_heads`` query/key heads serve ``heads`` value heads (head h uses h // (heads / qk_heads)).  The state S starts
at zero, is float32 and belongs to the request, as do the convolutions' last ``taps - 1`` inputs
(:class:`~hfee_b200.cache.CacheBundle` of two :class:`~hfee_b200.cache.FixedState`), so a request continues from
whatever portion came before.  Each head's read-out is RMS-normed over ``value_dim`` with one weight vector for
all heads, multiplied by silu(W_g x) and projected by W_o.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..cache.needs import CacheBundle, FixedState
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Mixer, register_part
from .gated_attention import pad8


class GatedDeltaRule(Mixer):
    """spec: ``width``, ``heads``, ``qk_heads``, ``key_dim``, ``value_dim``, ``taps``, ``eps`` (of the output norm)."""
    graph_safe = True
    can_overwrite = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        qk, vg = spec.qk_heads * spec.key_dim, spec.heads * spec.value_dim
        return {"q": TensorNeed((qk, spec.width)), "k": TensorNeed((qk, spec.width)), "v": TensorNeed((vg, spec.width)),
                "q_conv": TensorNeed((qk, spec.taps), role="vector"), "k_conv": TensorNeed((qk, spec.taps), role="vector"),
                "v_conv": TensorNeed((vg, spec.taps), role="vector"),
                "b": TensorNeed((spec.heads, spec.width)), "a": TensorNeed((spec.heads, spec.width)),
                "A_log": TensorNeed((spec.heads,), role="vector"), "dt_bias": TensorNeed((spec.heads,), role="vector"),
                "norm": TensorNeed((spec.value_dim,), role="scale"), "g": TensorNeed((vg, spec.width)),
                "o": TensorNeed((spec.width, vg))}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.qk_heads = int(spec.heads), int(spec.qk_heads)
        if self.heads % self.qk_heads:
            raise ValueError(f"heads {self.heads} must be a multiple of qk_heads {self.qk_heads}")
        self.key_dim, self.value_dim, self.taps = int(spec.key_dim), int(spec.value_dim), int(spec.taps)
        if self.taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {self.taps}")
        self.eps = float(spec.eps)
        self.qk_cols, self.vg_cols = self.qk_heads * self.key_dim, self.heads * self.value_dim
        self.conv_cols = 2 * self.qk_cols + self.vg_cols
        # one fused projection: rows [q | k | v | g | b | a]; the convolution runs over the first three at once
        self.w_in = torch.cat([tensors[k] for k in ("q", "k", "v", "g", "b", "a")], dim=0).contiguous()
        self.in_cols = self.w_in.shape[0]
        self.g_at = self.conv_cols
        self.b_at = self.g_at + self.vg_cols
        self.a_at = self.b_at + self.heads
        self.conv_weight = torch.cat([tensors["q_conv"], tensors["k_conv"], tensors["v_conv"]], dim=0).contiguous()
        self.a_log, self.dt_bias = tensors["A_log"], tensors["dt_bias"]
        self.norm_weight = tensors["norm"]
        self.w_o = tensors["o"]

    def cache_need(self) -> CacheBundle:
        return CacheBundle.of(None, conv=FixedState((self.taps - 1, self.conv_cols), "float32"),
                              recurrent=FixedState((self.heads, self.key_dim, self.value_dim), "float32"))

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: Any, cache: Any, writes_cache: bool,
                accumulate: bool = True) -> None:
        n, rt = step.n, self.rt
        x = x if isinstance(x, torch.Tensor) else x.tensor()
        proj = rt.scratch("delta_proj", (rt.max_tokens, pad8(self.in_cols)))[:n, :self.in_cols]
        ops.tag("qkv")
        ops.linear(x, self.w_in, proj)
        qkv = rt.scratch("delta_conv", (rt.max_tokens, pad8(self.conv_cols)))[:n, :self.conv_cols]
        ops.tag("conv")
        ops.conv_act(proj[:, :self.conv_cols], self.conv_weight, cache.states["conv"], step, qkv, "silu", writes_cache)
        o = rt.scratch("delta_out", (rt.max_tokens, self.vg_cols), torch.float32)[:n]
        ops.tag("delta_rule")
        workspace = None
        if step.max_new > 1:
            # the state-independent part of every tile of 16 tokens; sized once for the engine's limits
            workspace = rt.scratch("delta_tiles", (ops.delta_rule_workspace(
                rt.max_requests, rt.max_tokens, self.heads, self.qk_heads, self.key_dim),), torch.float32)
        ops.delta_rule(qkv, 0, self.qk_cols, 2 * self.qk_cols, proj, self.b_at, self.a_at, self.a_log, self.dt_bias,
                       cache.states["recurrent"], step, o, self.heads, self.qk_heads, self.key_dim, self.value_dim,
                       writes_cache, workspace)
        gated = rt.scratch("delta_gated", (rt.max_tokens, pad8(self.vg_cols)))[:n, :self.vg_cols]
        ops.tag("gate")
        ops.head_norm_gate(o, self.norm_weight, self.eps, proj[:, self.g_at:self.g_at + self.vg_cols], gated, self.heads,
                           self.value_dim, "silu")
        ops.tag("o")
        ops.linear(gated, self.w_o, out, accumulate=accumulate)


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
