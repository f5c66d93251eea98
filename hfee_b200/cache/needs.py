"""What a mixer asks of the cache manager for one request."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class PagedKV:
    """Keys and values for every cached position (or, with ``window``, for the last
    ``window`` positions only; with ``chunk``, for the positions of the current block of
    ``chunk`` positions counted from 0 only), stored in pages of ``page_size`` tokens.
    ``value_dim``: size of a cached value; None = ``head_dim``; 0 = nothing is cached beside the keys (the
    values are read out of the cached keys, as with a latent that serves as both)."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    chunk: Optional[int] = None
    value_dim: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """A per-request state of fixed size (``shape`` elements of ``dtype``), zeroed
    when the request is admitted."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class CacheBundle:
    """What a layer with several stateful parts asks for: at most one :class:`PagedKV` and any number of
    named :class:`FixedState` (a short convolution's history beside a recurrent state, say).  The view
    the layer gets has the pages as usual and ``states[name]`` per named state."""
    paged: Optional[PagedKV] = None
    states: Tuple[Tuple[str, FixedState], ...] = ()

    @classmethod
    def of(cls, paged: Optional[PagedKV] = None, **states: FixedState) -> "CacheBundle":
        return cls(paged, tuple(sorted(states.items())))

    def state_map(self) -> Dict[str, FixedState]:
        return dict(self.states)
