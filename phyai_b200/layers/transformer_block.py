"""One configurable pre-norm (or sandwich-norm) transformer block.

Covers the decoder / encoder blocks of the served families through configuration instead
of one class per model: attention kind (``attention`` no cache, ``ar`` / ``diffusion`` paged),
RMSNorm / Gemma RMSNorm / LayerNorm, optional per-head q/k RMSNorm, optional RoPE, gated or
plain MLP, biases, and checkpoint sub-key names for Llama / Qwen2 / Qwen3 / Gemma 1-3 /
SigLIP. Reference: phyai/src/phyai/layers/transformer_block.py:201-766.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from ..engine_config import resolve_engine_defaults
from ..ops import ref
from .attention import ARAttention, Attention, DiffusionAttention, PagedAttnCtx, RaggedMeta
from .layer_norm import GemmaRMSNorm, LayerNorm, RMSNorm
from .linear import QKVParallelLinear, RowParallelLinear
from .mlp import DenseMLP
from .rotary_embedding import RotaryEmbedding


@dataclass(frozen=True)
class BlockNames:
    """Checkpoint sub-keys of one block."""

    input_norm: str = "input_layernorm"
    post_attn_norm: str = "post_attention_layernorm"
    pre_mlp_norm: str | None = None          # sandwich norms (Gemma 2/3)
    post_mlp_norm: str | None = None
    attn: str = "self_attn"
    attn_out: str = "o_proj"
    q_norm: str = "q_norm"
    k_norm: str = "k_norm"
    mlp: str = "mlp"
    mlp_legs: tuple[str, ...] | None = None


LLAMA_NAMES = BlockNames()
QWEN2_NAMES = BlockNames()
QWEN3_NAMES = BlockNames()
GEMMA_NAMES = BlockNames()
GEMMA2_NAMES = BlockNames(pre_mlp_norm="pre_feedforward_layernorm", post_mlp_norm="post_feedforward_layernorm")
GEMMA3_NAMES = GEMMA2_NAMES
SIGLIP_NAMES = BlockNames(input_norm="layer_norm1", post_attn_norm="layer_norm2", attn_out="out_proj",
                          mlp_legs=("fc1", "fc2"))
SIGLIP_NORM_HF_NAMES = ("layer_norm1", "layer_norm2")

_NORMS = {"rmsnorm": RMSNorm, "gemma_rmsnorm": GemmaRMSNorm, "layernorm": LayerNorm}


class TransformerBlock(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, intermediate_size: int, *,
                 num_kv_heads: int | None = None, layer_id: int = 0, attn_kind: str = "attention",
                 attn_causal: bool = False, attn_bias: bool = False, attn_out_bias: bool = False,
                 sliding_window: int | None = None, logits_soft_cap: float | None = None, qk_norm: bool = False,
                 rope: RotaryEmbedding | None = None, mlp_gated: bool = True, mlp_activation: str = "silu",
                 mlp_bias: bool = False, norm_type: str = "rmsnorm", norm_eps: float = 1e-6, sandwich_norm: bool = False,
                 names: BlockNames = LLAMA_NAMES, attn_backend: str | None = None, norm_backend: str | None = None,
                 params_dtype: torch.dtype | None = None, prefix: str = "") -> None:
        super().__init__()
        dtype, attn_backend, norm_backend = resolve_engine_defaults(params_dtype, attn_backend, norm_backend)
        if norm_type not in _NORMS:
            raise ValueError(f"norm_type must be one of {sorted(_NORMS)}")
        Norm = _NORMS[norm_type]
        pre = (prefix + ".") if prefix else ""
        self.head_dim, self.rope, self.names = head_dim, rope, names
        nk = dict(backend=norm_backend, dtype=dtype)
        self.input_norm = Norm(hidden_size, norm_eps, prefix=pre + names.input_norm, **nk)
        self.post_attn_norm = Norm(hidden_size, norm_eps, prefix=pre + names.post_attn_norm, **nk)
        self.sandwich = sandwich_norm
        if sandwich_norm:
            self.pre_mlp_norm = Norm(hidden_size, norm_eps, prefix=pre + (names.pre_mlp_norm or "pre_feedforward_layernorm"), **nk)
            self.post_mlp_norm = Norm(hidden_size, norm_eps, prefix=pre + (names.post_mlp_norm or "post_feedforward_layernorm"), **nk)
        ap = pre + names.attn
        self.qkv_proj = QKVParallelLinear(hidden_size, head_dim, num_heads, num_kv_heads, bias=attn_bias,
                                          params_dtype=dtype, prefix=f"{ap}.qkv_proj")
        self.o_proj = RowParallelLinear(num_heads * head_dim, hidden_size, bias=attn_out_bias, params_dtype=dtype,
                                        prefix=f"{ap}.{names.attn_out}")
        self.qk_norm = qk_norm
        if qk_norm:
            self.q_norm = RMSNorm(head_dim, norm_eps, prefix=f"{ap}.{names.q_norm}", **nk)
            self.k_norm = RMSNorm(head_dim, norm_eps, prefix=f"{ap}.{names.k_norm}", **nk)
        hq, hkv = self.qkv_proj.num_heads, self.qkv_proj.num_kv_heads
        if attn_kind == "attention":
            self.attn = Attention(hq, head_dim, hkv, causal=attn_causal, sliding_window=sliding_window,
                                  logits_soft_cap=logits_soft_cap, backend=attn_backend)
        elif attn_kind == "ar":
            self.attn = ARAttention(layer_id, hq, head_dim, hkv, causal=attn_causal, backend=attn_backend)
        elif attn_kind == "diffusion":
            self.attn = DiffusionAttention(layer_id, hq, head_dim, hkv, causal=attn_causal, backend=attn_backend)
        else:
            raise ValueError(f"attn_kind {attn_kind!r}: expected attention / ar / diffusion")
        self.attn_kind = attn_kind
        self.mlp = DenseMLP(hidden_size, intermediate_size, gated=mlp_gated, activation=mlp_activation, bias=mlp_bias,
                            params_dtype=dtype, prefix=pre + names.mlp, hf_names=names.mlp_legs)

    def _qkv(self, x: torch.Tensor):
        qkv, _ = self.qkv_proj(x)
        p = self.qkv_proj
        q, k, v = qkv.split([p.q_size, p.kv_size, p.kv_size], dim=-1)
        lead = x.shape[:-1]
        q = q.reshape(*lead, p.num_heads, self.head_dim)
        k = k.reshape(*lead, p.num_kv_heads, self.head_dim)
        v = v.reshape(*lead, p.num_kv_heads, self.head_dim)
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        return q, k, v

    def forward(self, h: torch.Tensor, *, position_ids: torch.Tensor | None = None, cos_sin: torch.Tensor | None = None,
                meta: RaggedMeta | None = None, ctx: PagedAttnCtx | None = None, mask: torch.Tensor | None = None) -> torch.Tensor:
        """``h``: (B, S, H) padded or (T, H) ragged/paged. RoPE comes from ``cos_sin`` (T, rot) when
        given, else from the block's ``rope`` at ``position_ids``."""
        x = self.input_norm(h)
        q, k, v = self._qkv(x)
        if cos_sin is None and self.rope is not None and position_ids is not None:
            cos_sin = self.rope.cos_sin_cache[position_ids.long()]
        if cos_sin is not None:
            shp_q, shp_k = q.shape, k.shape
            q = ref.apply_rope(q.reshape(-1, *shp_q[-2:]), cos_sin.reshape(-1, cos_sin.shape[-1])).reshape(shp_q)
            k = ref.apply_rope(k.reshape(-1, *shp_k[-2:]), cos_sin.reshape(-1, cos_sin.shape[-1])).reshape(shp_k)
        if self.attn_kind == "attention":
            a = self.attn(q, k, v, meta=meta, mask=mask)
        else:
            if ctx is None:
                raise ValueError("paged attention needs a PagedAttnCtx")
            a = self.attn(q, k, v, ctx)
        a, _ = self.o_proj(a.reshape(*h.shape[:-1], -1))
        if self.sandwich:
            h = h + self.post_attn_norm(a)
            return h + self.post_mlp_norm(self.mlp(self.pre_mlp_norm(h)))
        h = h + a
        return h + self.mlp(self.post_attn_norm(h))


__all__ = ["TransformerBlock", "BlockNames", "LLAMA_NAMES", "QWEN2_NAMES", "QWEN3_NAMES", "GEMMA_NAMES",
           "GEMMA2_NAMES", "GEMMA3_NAMES", "SIGLIP_NAMES", "SIGLIP_NORM_HF_NAMES"]
