"""Token pool of a latent-attention model: ONE row [c | kr] per token and layer, shared by all heads
(c: the normed KV latent, kr: the rotated shared key part).  Same indexing as MHATokenToKVPool — slot
ids from the token allocator, slot 0..page_size-1 is the dummy page — so ReqToTokenPool and the
paged allocator are used unchanged.  Layers that read another layer's latent own no buffer: they
alias their source's."""
from __future__ import annotations

from typing import Dict, Optional

import torch


class LatentTokenToKVPool:
    def __init__(self, size: int, page_size: int, dtype: torch.dtype, row_dims: Dict[int, int],
                 source_of: Dict[int, int], device: str):
        """row_dims: {layer that owns a buffer: kv_rank + rot_dim}; source_of: {layer: owning layer}."""
        self.size, self.page_size, self.dtype, self.device = size, page_size, dtype, device
        self.source_of = dict(source_of)
        self.kv_buffer = {l: torch.zeros((size + page_size, d), dtype=dtype, device=device)
                          for l, d in row_dims.items()}
        for l, src in self.source_of.items():
            if src not in self.kv_buffer:
                raise ValueError(f"layer {l} reads the latent of layer {src}, which owns none")

    def get_kv_buffer(self, layer_id: int) -> torch.Tensor:
        return self.kv_buffer[self.source_of.get(layer_id, layer_id)]

    def owns(self, layer_id: int) -> bool:
        return layer_id in self.kv_buffer

    def get_kv_size_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv_buffer.values())


class SeqStatePool:
    """Per-sequence carry of layers whose output at a token depends on the token before it (token
    shift, and any other fixed-size recurrent state): state[layer] is [slots, width] fp32, the slot is
    the sequence's row in ReqToTokenPool, so it is taken and given back with it.  Nothing is
    cleared on reuse: a kernel that reads the state of a token at position 0 substitutes zeros."""

    def __init__(self, slots: int, widths: Dict[int, int], device: str):
        self.slots = slots
        self.state = {l: torch.zeros((slots, w), dtype=torch.float32, device=device)
                      for l, w in widths.items()}

    def get(self, layer_id: int) -> Optional[torch.Tensor]:
        return self.state.get(layer_id)

    def size_bytes(self) -> int:
        return sum(t.numel() * 4 for t in self.state.values())
