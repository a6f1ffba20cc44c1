"""What a mixer asks of the cache."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KVRequirement:
    """Keys and values of every position (window None) or of the last ``window`` positions.
    ``shared_values``: one tensor serves as both (a layer that caches a single vector a token, from
    which it derives keys and values); ``view.v`` is then ``view.k``.  ``chunk``: a query reads only
    the keys of its own block of that many positions (blocks counted from position 0), so the pages
    of earlier blocks come back as the sequence grows.  ``keep_first``: beside its window a query
    reads the keys at positions below this, so the pages that hold any of them are never given back."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    shared_values: bool = False
    chunk: Optional[int] = None
    keep_first: int = 0

    @property
    def kept_pages(self) -> int:
        """How many pages at the start of a sequence a window never releases (pages of 64 tokens)."""
        return (self.keep_first + 63) // 64 if self.releases else 0

    def first_needed(self, length: int) -> int:
        """The lowest position that a query at position >= ``length`` can still read (0: everything stays)."""
        if self.window is not None:
            return max(0, length - self.window + 1)
        if self.chunk is not None:
            return length - length % self.chunk
        return 0

    @property
    def releases(self) -> bool:
        return self.window is not None or self.chunk is not None

    @property
    def span(self) -> Optional[int]:
        """The most positions behind a query that it can read, when that is bounded."""
        return self.window if self.window is not None else self.chunk


@dataclass(frozen=True)
class StateRequirement:
    """A tensor of fixed shape per sequence, zero when the sequence starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class BundleRequirement:
    """What a layer asks when it keeps more than one thing a sequence: ``main`` (keys and values, a state, or None)
    and named states of fixed shape beside it (the last inputs of a short convolution, the row of the token
    before).  The layer's view of the cache then has ``extras[name]``, a state view of its own, for each."""

    main: object
    extras: Tuple[Tuple[str, StateRequirement], ...] = ()

    @staticmethod
    def of(main, **extras) -> "BundleRequirement":
        """``main`` may itself be a bundle: its states are kept, the new ones join them."""
        have = ()
        if isinstance(main, BundleRequirement):
            main, have = main.main, main.extras
        names = [n for n, _ in have]
        for n in extras:
            if n in names:
                raise ValueError(f"two states of one layer are called {n!r}")
        return BundleRequirement(main, tuple(have) + tuple(sorted(extras.items())))


def simple_requirements(req):
    """The requirements a layer's answer is made of, one by one (a bundle: its main one, then its states)."""
    if isinstance(req, BundleRequirement):
        return ([req.main] if req.main is not None else []) + [st for _, st in req.extras]
    return [] if req is None else [req]
