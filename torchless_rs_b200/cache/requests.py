"""What a mixer asks of the cache.  A mixer names its need; the cache groups
layers with equal needs and gives each group storage of its own."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class PagedKVRequest:
    """Keys and values of every position (window None), or of the last `window`
    positions only; with `keep_first`, the sequence's first `keep_first` positions stay
    visible (and held) whatever the window.  `v_head_dim`: the size of a value where it is
    not the size of a key."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None
    keep_first: int = 0

    @property
    def value_dim(self) -> int:
        return self.v_head_dim if self.v_head_dim else self.head_dim


@dataclass(frozen=True)
class PagedLatentRequest:
    """One vector of `width` numbers per position, shared by all heads (the compressed keys
    and values of latent attention), of every position or of the last `window` only."""
    width: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """Per-sequence state of fixed size, zero when a sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
