"""RecurrentCache: per-layer recurrent states with the interface of mmfreelm/models/utils.py:11-104."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

try:  # keep isinstance(cache, transformers.Cache) true where that class can be subclassed freely
    from transformers.cache_utils import Cache as _HFCache
except Exception:  # pragma: no cover
    _HFCache = object


class RecurrentCache(_HFCache):
    """List of per-layer state tuples; the first `update` of a layer stores the tuple, later ones copy into
    it in place, and the token tally advances when the last layer is updated."""

    def __init__(self, seen_tokens: int = 0):
        # deliberately no super().__init__(): the HF base class wants layer objects this cache does not use
        self.states: List[Tuple[torch.Tensor, ...]] = []
        self._seen_tokens = seen_tokens

    def __getitem__(self, layer_idx: int):
        if layer_idx < len(self):
            return self.states[layer_idx]
        raise KeyError(f"Cache only has {len(self)} layers, attempted to access layer with index {layer_idx}")

    def __iter__(self):
        yield from self.states

    def __len__(self):
        return len(self.states)

    def update(self, state, layer_idx: int, cache_kwargs: Optional[Dict[str, Any]] = None):
        if isinstance(state, torch.Tensor):
            state = (state,)
        if len(self.states) <= layer_idx:
            self.states.append(tuple(state))
        else:
            for dst, src in zip(self.states[layer_idx], state):
                if dst.data_ptr() != src.data_ptr():
                    dst.copy_(src)
            if layer_idx == len(self) - 1:
                self._seen_tokens += 1
        return state

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        return 0 if len(self.states) <= layer_idx else self._seen_tokens

    def get_max_length(self) -> Optional[int]:
        return None

    def reorder_cache(self, beam_idx: torch.LongTensor):
        self.states = [tuple(s.index_select(0, beam_idx.to(s.device)) for s in layer) for layer in self.states]

    def to_legacy_cache(self):
        return tuple(self.states)

    @classmethod
    def from_legacy_cache(cls, past_key_values=None, seen_tokens: int = 0) -> "RecurrentCache":
        cache = cls(seen_tokens)
        if past_key_values is not None:
            for layer_idx, state in enumerate(past_key_values):
                cache.update(state, layer_idx)
        return cache
