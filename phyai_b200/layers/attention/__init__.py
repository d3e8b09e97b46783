from .common import AttnLayout, AttnMode, RaggedMeta, build_padded_mask, eager_attn, repeat_kv
from .layers import (ARAttention, ARAttnCtx, ARAttnMetadata, Attention, DiffusionAttention, DiffusionAttnCtx,
                     DiffusionAttnMetadata, PagedAttnCtx, PagedAttnMetadata)

__all__ = ["AttnLayout", "AttnMode", "RaggedMeta", "build_padded_mask", "eager_attn", "repeat_kv", "ARAttention",
           "ARAttnCtx", "ARAttnMetadata", "Attention", "DiffusionAttention", "DiffusionAttnCtx", "DiffusionAttnMetadata",
           "PagedAttnCtx", "PagedAttnMetadata"]
