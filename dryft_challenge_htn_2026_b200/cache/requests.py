"""What a mixer asks of the cache. Entries with equal requests share one group (one storage)."""
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KVRequest:
    """Keys and values per token: [n_kv_heads, head_dim] each (values [n_kv_heads, v_head_dim] when
    that is given and differs: the two then live in stores of their own). ``window``: only the last
    ``window`` tokens are ever read, older pages may be given back; None: all tokens are kept.
    ``chunk``: a token reads only keys of its own chunk of that many positions (counted from the
    sequence's start), so pages wholly before the chunk of the next token may be given back.
    ``keep_first``: the first that many positions stay in sight whatever the window or chunk: their pages
    are never given back. ``values_in_keys``: a token's value row is the first ``v_head_dim`` numbers of its key row
    (rows of latents): there is no store of values, and a view's ``v`` is None."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int]
    dtype: torch.dtype
    v_head_dim: Optional[int] = None
    chunk: Optional[int] = None
    keep_first: int = 0
    values_in_keys: bool = False


@dataclass(frozen=True)
class StateRequest:
    """A state of fixed shape per sequence, zero when the sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype
