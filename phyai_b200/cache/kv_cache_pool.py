"""Paged KV pool with page size 1.

One K and one V tensor for all layers, shape ``(layers, slots, kv_heads, head_dim)``;
slot 0 is a sentinel that padding rows write to and nobody reads. ``write_kv`` is a
pure index scatter; on the CUDA path the scatter is fused into the RoPE kernel
(``ops.rope_kv``) and this method is only the reference. Reference:
phyai/src/phyai/cache/kv_cache_pool.py:31-269.
"""

from __future__ import annotations

import torch


class KVCachePool:
    def __init__(self, num_layers: int, num_slots: int, num_kv_heads: int, head_dim: int, *,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device | str = "cuda", page_size: int = 1) -> None:
        if page_size != 1:
            raise ValueError("KVCachePool supports page_size=1 only")
        if min(num_layers, num_slots, num_kv_heads, head_dim) <= 0:
            raise ValueError("KVCachePool: all sizes must be positive")
        self.num_layers, self.num_slots = num_layers, num_slots
        self.num_kv_heads, self.head_dim, self.page_size = num_kv_heads, head_dim, page_size
        self.dtype, self.device = dtype, torch.device(device)
        shape = (num_layers, num_slots, num_kv_heads, head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=self.device)
        self.v = torch.zeros(shape, dtype=dtype, device=self.device)

    def layer(self, layer_id: int) -> tuple[torch.Tensor, torch.Tensor]:
        """``(slots, kv_heads, head_dim)`` views of one layer."""
        return self.k[layer_id], self.v[layer_id]

    def k_buffer(self, layer_id: int) -> torch.Tensor:
        """The layer's K rows ``(slots, kv_heads, head_dim)``: a view of the pool, writes through it reach the pool."""
        return self.k[layer_id]

    def v_buffer(self, layer_id: int) -> torch.Tensor:
        return self.v[layer_id]

    def kv_buffer(self, layer_id: int) -> tuple[torch.Tensor, torch.Tensor]:
        return self.k[layer_id], self.v[layer_id]

    def write_kv(self, layer_id: int, k: torch.Tensor, v: torch.Tensor, write_indices: torch.Tensor) -> None:
        """Scatter ``k``/``v`` rows ``(T, kv_heads, head_dim)`` to the slots in ``write_indices`` (int64)."""
        if write_indices.dtype != torch.int64:
            raise TypeError("write_indices must be int64")
        self.k[layer_id].index_copy_(0, write_indices, k.to(self.dtype))
        self.v[layer_id].index_copy_(0, write_indices, v.to(self.dtype))

    def gather_kv(self, layer_id: int, indices: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        idx = indices.long()
        return self.k[layer_id][idx], self.v[layer_id][idx]

    def zero_(self) -> None:
        self.k.zero_()
        self.v.zero_()

    @property
    def total_bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


__all__ = ["KVCachePool"]
