from .common import AttnLayout, AttnMode, RaggedMeta, build_padded_mask, eager_attn, repeat_kv
from .gdn import (GDN_BACKENDS, GatedDeltaNet, GatedDeltaNetAttention, GatedDeltaNetCtx, gated_delta_rule_chunked,
                  gated_delta_rule_recurrent, list_gdn_backends)
from .layers import (ARAttention, ARAttnCtx, ARAttnMetadata, Attention, DiffusionAttention, DiffusionAttnCtx,
                     DiffusionAttnMetadata, PagedAttnCtx, PagedAttnMetadata)

AttnMetadata, AttnCtx = PagedAttnMetadata, PagedAttnCtx      # the names of the reference's paged layers
ATTENTION_BACKENDS = ("b200", "torch")


def list_attention_backends() -> list[str]:
    """Backends of :class:`Attention` (``"b200"``: the tcgen05 kernel, ``"torch"``: SDPA / eager); the paged layers take the same."""
    return list(ATTENTION_BACKENDS)


list_ar_backends = list_diffusion_backends = list_attention_backends

__all__ = ["GatedDeltaNet", "GatedDeltaNetAttention", "GatedDeltaNetCtx", "GDN_BACKENDS", "list_gdn_backends", "gated_delta_rule_chunked",
           "gated_delta_rule_recurrent", "AttnMetadata", "AttnCtx", "ATTENTION_BACKENDS", "list_attention_backends", "list_ar_backends",
           "list_diffusion_backends", "AttnLayout", "AttnMode", "RaggedMeta", "build_padded_mask", "eager_attn", "repeat_kv", "ARAttention",
           "ARAttnCtx", "ARAttnMetadata", "Attention", "DiffusionAttention", "DiffusionAttnCtx", "DiffusionAttnMetadata",
           "PagedAttnCtx", "PagedAttnMetadata"]
