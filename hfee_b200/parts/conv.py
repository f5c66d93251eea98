"""Short causal convolution over time, added to its input: what a mixer reads is ``x + conv(x)``.

``conv(x)[t] = sum_j w[:, j] * x[t - taps + 1 + j]`` per channel, with zeros in front of a
request's first token.  The last ``taps - 1`` inputs of every request are a state of their own
(:class:`~hfee_b200.cache.FixedState`), so a prompt may be cut anywhere and decoding continues it.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..cache.needs import FixedState
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Part, register_part


class CausalDepthwiseConv(Part):
    """spec: ``width``, ``taps``.  Tensor ``weight`` [width, taps] (float32 on the device)."""
    category = "conv"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"weight": TensorNeed((spec.width, spec.taps), role="vector")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.width, self.taps = int(spec.width), int(spec.taps)
        if self.taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {self.taps}")
        self.weight = tensors["weight"]

    def cache_need(self) -> FixedState:
        return FixedState((self.taps - 1, self.width), "float32")

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: Any, state: torch.Tensor, write_state: bool = True) -> None:
        """``out = x + conv(x)`` for the step's tokens; ``state`` [slots, taps - 1, width] is read and renewed."""
        before = ops.tag("conv")
        ops.short_conv(x, self.weight, state, step, out, write_state)
        ops.tag(before)


register_part("conv", "causal_depthwise", CausalDepthwiseConv)
