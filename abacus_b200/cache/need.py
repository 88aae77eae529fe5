"""What a mixer asks of the cache for one entry of the schedule."""
from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class CacheNeed:
    """Per-token keys and values (n_kv_heads > 0), all of them or a window of the last ones,
    and/or a per-sequence state of fixed shape (float32, zeroed when a slot is handed out).

    v_head_dim: the size of a value head where it is not head_dim. keep_first (with a window): the sequence's
    first keep_first tokens are kept for good beside the window. values_in_keys: a value is the first v_head_dim
    elements of its key row, and the group has one pool for both. states: further per-sequence states by name,
    ((name, shape, "float32" or "int32"), ...), zeroed like the first."""
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    v_head_dim: Optional[int] = None
    keep_first: int = 0
    states: Tuple[tuple, ...] = ()
    values_in_keys: bool = False
