"""What a mixer asks of the cache manager."""
from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class CacheNeed:
    """kind "paged_kv": keys and values of every position (or of the last
    `window` positions) in pages; kind "state": one block of fixed shape per
    request.  Calls whose needs are equal share a group: one page id (or slot
    id) is valid in all of them.  `shared` (paged_kv): a position keeps ONE row
    per head that is read as key and as value (a latent from which a mixer makes
    both), so a page holds half as much.  `v_dim` (paged_kv): values of another size than the
    keys' `head_dim`; a page is then one flat block, n_kv_heads x page_size x head_dim keys followed
    by n_kv_heads x page_size x v_dim values.  `chunk` (paged_kv): a query sees only keys of its own
    chunk of so many positions (counted from position 0), so pages of earlier chunks go back to the
    pool as a window's do.  A mixer with several things to keep answers with a tuple of needs and
    gets a tuple of bindings."""
    kind: str
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"
    shared: bool = False
    v_dim: Optional[int] = None
    chunk: Optional[int] = None

    @classmethod
    def paged_kv(cls, n_kv_heads, head_dim, window=None, shared=False, v_dim=None, chunk=None):
        if window is not None and window <= 0:
            raise ValueError("window must be a positive count of keys or None")
        if chunk is not None and chunk <= 0:
            raise ValueError("chunk must be a positive count of positions or None")
        if v_dim is not None and (shared or v_dim <= 0):
            raise ValueError("v_dim must be positive and does not go with shared rows")
        return cls("paged_kv", int(n_kv_heads), int(head_dim), None if window is None else int(window),
                   shared=bool(shared), v_dim=None if v_dim is None else int(v_dim),
                   chunk=None if chunk is None else int(chunk))

    @classmethod
    def state(cls, shape, dtype="float32"):
        return cls("state", state_shape=tuple(int(s) for s in shape), state_dtype=dtype)


@dataclass
class CacheBinding:
    """What a mixer call gets: its own tensor and the group whose block tables
    (or slot ids) index it.  paged_kv: tensor [n_pages, 2, n_kv_heads,
    page_size, head_dim] ([n_pages, 1, ...] for a shared need; [n_pages, n_kv_heads * page_size *
    (head_dim + v_dim)] for a need with v_dim); state: tensor
    [n_slots, *state_shape].  `write` is
    false for a call that reads the cache another call wrote."""
    kind: str
    group: int
    tensor: object
    write: bool = True
