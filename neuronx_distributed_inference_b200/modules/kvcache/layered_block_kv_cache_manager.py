"""Paged KV cache whose layers may differ in shape or share storage, plus per-sequence state lines.

:class:`BlockKVCacheManager` keeps one ``[layers, 2, blocks, page, H, D]`` allocation, which fixes one head count and one head size for
every layer and gives every layer its own keys and values.  Hybrid stacks break all three assumptions: attention layers may have
different head counts, key and value sizes may differ (``D != Dv``), some layers have no cache at all (recurrent mixers) and some read
the cache of an earlier layer instead of writing one; latent attention keeps ONE row per token that serves as key and as value.  Here
every OWNING layer gets its own pair ``[blocks, page, H, D]`` /
``[blocks, page, H, Dv]``; a layer listed in ``share`` resolves to its source's pair; the block table is common to all layers, so
one page index names the same token range everywhere.  ``states`` (a :class:`RecurrentStateCache`) holds what is carried per
SEQUENCE rather than per token — convolution tails and recurrent states — in ``num_slots`` lines plus one scratch line that padded
batch rows are pointed at.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .recurrent_state_cache import RecurrentStateCache


class LayeredBlockKVCacheManager(nn.Module):
    def __init__(self, layer_shapes: Dict[int, Tuple[int, int, int]], share: Dict[int, int], num_blocks: int, block_size: int,
                 dtype=torch.bfloat16, device=None, state_specs: Optional[dict] = None, num_slots: int = 0, state_dtype=None):
        """``layer_shapes``: owning layer -> (kv heads, key size, value size); a value size of ``None`` makes the value tensor the key
        tensor itself (latent caches).  ``share``: reading layer -> owning layer.  "Layer" is whatever the model indexes its caches
        by: a stack that runs some layers several times gives every RUN its own entry."""
        super().__init__()
        self.num_blocks, self.block_size, self.num_slots = num_blocks, block_size, num_slots
        self.share = dict(share)
        for reader, owner in self.share.items():
            if owner not in layer_shapes:
                raise ValueError(f"layer {reader} reads the cache of layer {owner}, which owns none")
        self._index = {}
        for n, (layer, (H, D, Dv)) in enumerate(sorted(layer_shapes.items())):
            self.register_buffer(f"k_{n}", torch.zeros(num_blocks, block_size, H, D, dtype=dtype, device=device), persistent=False)
            if Dv is not None:
                self.register_buffer(f"v_{n}", torch.zeros(num_blocks, block_size, H, Dv, dtype=dtype, device=device), persistent=False)
            self._index[layer] = n
        self.states = RecurrentStateCache(state_specs or {}, num_slots, state_dtype or dtype, device)
        # the base model's bookkeeping expects these two names
        self.num_lines, self.garbage = num_slots, 1

    def owner_of(self, layer: int) -> int:
        return self.share.get(layer, layer)

    def get_kv_by_layer_id(self, idx: int):
        n = self._index[self.owner_of(idx)]
        k = getattr(self, f"k_{n}")
        return k, getattr(self, f"v_{n}", k)

    def lines_for(self, seq_ids: torch.Tensor) -> torch.Tensor:
        """State line of every batch row; rows without a sequence (negative id) use the scratch line."""
        bad = (seq_ids < 0) | (seq_ids >= self.num_slots)
        return torch.where(bad, torch.full_like(seq_ids, self.num_slots), seq_ids)

    def reset(self):
        for b in self.buffers():
            b.zero_()

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.buffers())
