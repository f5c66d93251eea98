"""Linear attention with a scalar decay per head, gated and normed on its way out.

Per head, with q, k of size ``key_dim`` and v of size ``value_dim`` (each an activation of a
projection of the mixer's input h)::

    S_t = decay_h * S_(t-1) + k_t v_t^T          o_t = S_t^T q_t

The state S starts at zero, is float32 and belongs to the request
(:class:`~hfee_b200.cache.FixedState`), so a request continues from whatever portion came before.
The heads' outputs are RMS-normed together, multiplied by ``sigmoid(W_g h)`` and projected by W_o.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..cache.needs import FixedState
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Mixer, register_part


class DecayLinearAttention(Mixer):
    """spec: ``width``, ``heads``, ``key_dim``, ``value_dim``, ``decay`` (one number per head),
    ``activation`` (``"silu"`` or ``"none"``, applied to q, k and v), ``eps`` (of the output norm).
    Tensors: ``q``, ``k`` [heads * key_dim, width], ``v``, ``g`` [heads * value_dim, width], ``o``
    [width, heads * value_dim], ``norm`` [heads * value_dim]."""
    graph_safe = True
    can_overwrite = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        qk, vg = spec.heads * spec.key_dim, spec.heads * spec.value_dim
        return {"q": TensorNeed((qk, spec.width)), "k": TensorNeed((qk, spec.width)),
                "v": TensorNeed((vg, spec.width)), "g": TensorNeed((vg, spec.width)),
                "o": TensorNeed((spec.width, vg)), "norm": TensorNeed((vg,), role="scale")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.key_dim, self.value_dim = int(spec.heads), int(spec.key_dim), int(spec.value_dim)
        decay = [float(d) for d in spec.decay]
        if len(decay) != self.heads:
            raise ValueError(f"{len(decay)} decays for {self.heads} heads")
        if any(not 0.0 <= d <= 1.0 for d in decay):
            raise ValueError(f"decays must lie in [0, 1], got {decay}")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=rt.device)
        self.activation = str(spec.get("activation", "silu"))
        self.eps = float(spec.eps)
        self.qk_cols, self.vg_cols = self.heads * self.key_dim, self.heads * self.value_dim
        # one fused projection: rows [q | k | v | g]
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0).contiguous()
        self.w_o = tensors["o"]
        self.norm_weight = tensors["norm"]
        self.in_cols = 2 * self.qk_cols + 2 * self.vg_cols

    def cache_need(self) -> FixedState:
        return FixedState((self.heads, self.key_dim, self.value_dim), "float32")

    def forward(self, h: torch.Tensor, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool,
                accumulate: bool = True) -> None:
        n, rt = step.n, self.rt
        h = h if isinstance(h, torch.Tensor) else h.tensor()
        state = cache.states["recurrent"] if cache.states else cache.state
        proj = rt.scratch("linattn_proj", (rt.max_tokens, self.in_cols))[:n]
        ops.tag("qkv")
        ops.linear(h, self.w_in, proj)
        a, b = self.qk_cols, 2 * self.qk_cols
        q, k, v, g = proj[:, :a], proj[:, a:b], proj[:, b:b + self.vg_cols], proj[:, b + self.vg_cols:]
        o = rt.scratch("linattn_out", (rt.max_tokens, self.vg_cols), torch.float32)[:n]
        ops.tag("linear_attention")
        workspace = None
        if step.max_new >= ops.LINEAR_ATTENTION_CHUNKED_MIN:
            # one state-sized sum per run of tokens; sized once for the engine's limits
            workspace = rt.scratch("linattn_runs", (ops.linear_attention_workspace(
                rt.max_requests, rt.max_tokens, self.heads, self.key_dim, self.value_dim),), torch.float32)
        ops.linear_attention(q, k, v, self.decay, state, step, o, self.heads, self.key_dim, self.value_dim,
                             self.activation, writes_cache, workspace)
        gated = rt.scratch("linattn_gated", (rt.max_tokens, self.vg_cols))[:n]
        ops.tag("gate")
        ops.norm_gate(o, self.norm_weight, self.eps, g, gated)
        ops.tag("o")
        ops.linear(gated, self.w_o, residual, accumulate=accumulate)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
