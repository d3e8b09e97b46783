"""Qwen3.5: a reference implementation (prefill only, replicated weights, not registered as a plugin).

Decoder layers alternate between gated delta-net (linear attention with a per-head matrix state:
short causal convolution over q|k|v, decay ``g = -exp(A_log) * softplus(a + dt_bias)``, write
strength ``beta = sigmoid(b)``, output RMS-normed and gated by ``silu(z)``) and full attention
whose query projection also emits a sigmoid output gate; rotary embedding covers only the first
``partial_rotary_factor`` of the head and is three-axis (mRoPE). The vision tower is the Qwen3-VL
one without DeepStack taps. Norm weights are stored zero-centred (the factor is ``1 + w``).

Reference: phyai/src/phyai/models/qwen3_5/modeling_qwen3_5.py:36-1361.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...layers.attention.gdn import GatedDeltaNetAttention
from ...layers.rotary_embedding import MRotaryEmbedding, rotate_half
from ..qwen3_vl.configuration_qwen3_vl import Qwen3VLVisionConfig
from ..qwen3_vl.modeling_qwen3_vl import Linear, Qwen3VLVisionModel, _key
from .configuration_qwen3_5 import Qwen3_5Config, Qwen3_5TextConfig


def qwen3_5_weight_remap(name: str) -> str | None:
    """Checkpoints carry a multi-token-prediction head this prefill-only model does not build."""
    return None if name.startswith("mtp.") else name


class ZeroCentredRMS(nn.Module):
    def __init__(self, d: int, eps: float, prefix: str, dtype=None, device=None) -> None:
        super().__init__()
        self.eps = eps
        self.weight = _key(nn.Parameter(torch.zeros(d, dtype=dtype, device=device)), f"{prefix}.weight")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * (1.0 + self.weight.float())).to(x.dtype)


class RMSNormGated(nn.Module):
    """``rms_norm(x) * w * silu(z)`` over the value head width."""

    def __init__(self, d: int, eps: float, prefix: str, dtype=None, device=None) -> None:
        super().__init__()
        self.eps = eps
        self.weight = _key(nn.Parameter(torch.ones(d, dtype=dtype, device=device)), f"{prefix}.weight")

    def forward(self, x: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()
        return (y * F.silu(z.float())).to(x.dtype)


class Qwen3_5GatedDeltaNet(nn.Module):
    def __init__(self, c: Qwen3_5TextConfig, prefix: str, **kw) -> None:
        super().__init__()
        self.c = c
        self.hk, self.hv, self.dk, self.dv = c.linear_num_key_heads, c.linear_num_value_heads, c.linear_key_head_dim, c.linear_value_head_dim
        self.key_dim, self.value_dim = self.hk * self.dk, self.hv * self.dv
        conv_dim = 2 * self.key_dim + self.value_dim
        H = c.hidden_size
        self.in_proj_qkv = Linear(H, conv_dim, bias=False, prefix=f"{prefix}.in_proj_qkv", **kw)
        self.in_proj_z = Linear(H, self.value_dim, bias=False, prefix=f"{prefix}.in_proj_z", **kw)
        self.in_proj_b = Linear(H, self.hv, bias=False, prefix=f"{prefix}.in_proj_b", **kw)
        self.in_proj_a = Linear(H, self.hv, bias=False, prefix=f"{prefix}.in_proj_a", **kw)
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, c.linear_conv_kernel_dim, groups=conv_dim, padding=c.linear_conv_kernel_dim - 1, bias=False, **kw)
        _key(self.conv1d.weight, f"{prefix}.conv1d.weight")
        self.A_log = _key(nn.Parameter(torch.zeros(self.hv, **kw)), f"{prefix}.A_log")
        self.dt_bias = _key(nn.Parameter(torch.ones(self.hv, **kw)), f"{prefix}.dt_bias")
        self.norm = RMSNormGated(self.dv, c.rms_norm_eps, f"{prefix}.norm", **kw)
        self.out_proj = Linear(self.value_dim, H, bias=False, prefix=f"{prefix}.out_proj", **kw)
        self.core = GatedDeltaNetAttention(self.hv, self.dk, self.dv)

    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
        B, S, _ = x.shape
        if mask is not None:
            x = x * mask[..., None].to(x.dtype)            # padding must not write into the state
        qkv = F.silu(self.conv1d(self.in_proj_qkv(x).transpose(1, 2))[:, :, :S]).transpose(1, 2)
        q, k, v = qkv.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        rep = self.hv // self.hk
        q = q.reshape(B, S, self.hk, self.dk).repeat_interleave(rep, dim=2)
        k = k.reshape(B, S, self.hk, self.dk).repeat_interleave(rep, dim=2)
        v = v.reshape(B, S, self.hv, self.dv)
        beta = torch.sigmoid(self.in_proj_b(x).float())
        g = -self.A_log.float().exp() * F.softplus(self.in_proj_a(x).float() + self.dt_bias.float())
        o = self.core.prefill(q, k, v, g, beta)
        z = self.in_proj_z(x).reshape(B, S, self.hv, self.dv)
        return self.out_proj(self.norm(o, z).reshape(B, S, self.value_dim))


class Qwen3_5Attention(nn.Module):
    def __init__(self, c: Qwen3_5TextConfig, prefix: str, **kw) -> None:
        super().__init__()
        self.c = c
        H, D, nq, nk = c.hidden_size, c.head_dim, c.num_attention_heads, c.num_key_value_heads
        self.q_proj = Linear(H, 2 * nq * D, bias=False, prefix=f"{prefix}.q_proj", **kw)     # per head: query | output gate
        self.k_proj, self.v_proj = Linear(H, nk * D, bias=False, prefix=f"{prefix}.k_proj", **kw), Linear(H, nk * D, bias=False, prefix=f"{prefix}.v_proj", **kw)
        self.o_proj = Linear(nq * D, H, bias=False, prefix=f"{prefix}.o_proj", **kw)
        self.q_norm, self.k_norm = ZeroCentredRMS(D, c.rms_norm_eps, f"{prefix}.q_norm", **kw), ZeroCentredRMS(D, c.rms_norm_eps, f"{prefix}.k_norm", **kw)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, mask: torch.Tensor | None) -> torch.Tensor:
        B, S, _ = x.shape
        c = self.c
        qg = self.q_proj(x).reshape(B, S, c.num_attention_heads, 2 * c.head_dim)
        q, gate = qg[..., :c.head_dim], qg[..., c.head_dim:]
        q = self.q_norm(q).transpose(1, 2)
        k = self.k_norm(self.k_proj(x).reshape(B, S, c.num_key_value_heads, c.head_dim)).transpose(1, 2)
        v = self.v_proj(x).reshape(B, S, c.num_key_value_heads, c.head_dim).transpose(1, 2)
        r = c.rotary_dim

        def rope(t):
            a, b = t[..., :r].float(), t[..., r:]
            return torch.cat([(a * cos[:, None] + rotate_half(a) * sin[:, None]).to(t.dtype), b], dim=-1)

        o = F.scaled_dot_product_attention(rope(q), rope(k), v, attn_mask=mask, is_causal=mask is None, enable_gqa=True)
        o = o.transpose(1, 2) * torch.sigmoid(gate.float()).to(o.dtype)
        return self.o_proj(o.reshape(B, S, -1))


class Qwen3_5DecoderLayer(nn.Module):
    def __init__(self, c: Qwen3_5TextConfig, kind: str, prefix: str, **kw) -> None:
        super().__init__()
        self.kind = kind
        self.input_layernorm = ZeroCentredRMS(c.hidden_size, c.rms_norm_eps, f"{prefix}.input_layernorm", **kw)
        self.post_attention_layernorm = ZeroCentredRMS(c.hidden_size, c.rms_norm_eps, f"{prefix}.post_attention_layernorm", **kw)
        if kind == "linear_attention":
            self.linear_attn = Qwen3_5GatedDeltaNet(c, f"{prefix}.linear_attn", **kw)
        else:
            self.self_attn = Qwen3_5Attention(c, f"{prefix}.self_attn", **kw)
        m = f"{prefix}.mlp"
        self.gate_proj = Linear(c.hidden_size, c.intermediate_size, bias=False, prefix=f"{m}.gate_proj", **kw)
        self.up_proj = Linear(c.hidden_size, c.intermediate_size, bias=False, prefix=f"{m}.up_proj", **kw)
        self.down_proj = Linear(c.intermediate_size, c.hidden_size, bias=False, prefix=f"{m}.down_proj", **kw)

    def forward(self, x, cos, sin, mask4, pad_mask):
        h = self.input_layernorm(x)
        x = x + (self.linear_attn(h, pad_mask) if self.kind == "linear_attention" else self.self_attn(h, cos, sin, mask4))
        h = self.post_attention_layernorm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class Qwen3_5TextModel(nn.Module):
    def __init__(self, c: Qwen3_5TextConfig, prefix: str = "model.language_model", **kw) -> None:
        super().__init__()
        self.c = c
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size, **kw)
        _key(self.embed_tokens.weight, f"{prefix}.embed_tokens.weight")
        self.layers = nn.ModuleList([Qwen3_5DecoderLayer(c, kind, f"{prefix}.layers.{i}", **kw) for i, kind in enumerate(c.layer_types)])
        self.norm = ZeroCentredRMS(c.hidden_size, c.rms_norm_eps, f"{prefix}.norm", **kw)
        self.rotary = MRotaryEmbedding(c.rotary_dim, c.mrope_section, c.rope_theta, interleaved=True)

    def forward(self, inputs_embeds: torch.Tensor, position_ids: torch.Tensor, attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        B, S, _ = inputs_embeds.shape
        cs = torch.stack([self.rotary.cos_sin(position_ids[:, b].float()) for b in range(B)])
        half = self.c.rotary_dim // 2
        cos, sin = cs[..., :half].repeat(1, 1, 2), cs[..., half:].repeat(1, 1, 2)
        mask4 = None
        if attention_mask is not None:
            mask4 = torch.ones(S, S, dtype=torch.bool, device=inputs_embeds.device).tril()[None, None] & attention_mask[:, None, None].bool()
        x = inputs_embeds
        for layer in self.layers:
            x = layer(x, cos, sin, mask4, attention_mask)
        return self.norm(x)


class Qwen3_5Model(nn.Module):
    def __init__(self, config: Qwen3_5Config, *, dtype=None, device=None) -> None:
        super().__init__()
        kw = {k: v for k, v in (("dtype", dtype), ("device", device)) if v is not None}
        self.config = config
        v = config.vision_config
        self.visual = Qwen3VLVisionModel(Qwen3VLVisionConfig(**{f: getattr(v, f) for f in (
            "depth", "hidden_size", "intermediate_size", "num_heads", "in_channels", "patch_size", "temporal_patch_size",
            "spatial_merge_size", "out_hidden_size", "num_position_embeddings", "deepstack_visual_indexes", "hidden_act")}), **kw)
        self.language_model = Qwen3_5TextModel(config.text_config, **kw)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, *, pixel_patches: torch.Tensor | None = None, grid_thw: torch.Tensor | None = None,
                attention_mask: torch.Tensor | None = None, position_ids: torch.Tensor | None = None) -> torch.Tensor:
        x = self.language_model.embed_tokens(input_ids)
        if pixel_patches is not None:
            feats, _ = self.visual(pixel_patches.to(x.dtype), grid_thw)
            where = (input_ids == self.config.image_token_id) | (input_ids == self.config.video_token_id)
            if int(where.sum()) != feats.shape[0]:
                raise ValueError(f"{int(where.sum())} placeholder tokens for {feats.shape[0]} visual features")
            x = x.clone()
            x[where] = feats.to(x.dtype)
        if position_ids is None:
            B, S = input_ids.shape
            position_ids = torch.arange(S, device=input_ids.device)[None, None].expand(3, B, S)
        return self.language_model(x, position_ids, attention_mask)


class Qwen3_5ForConditionalGeneration(nn.Module):
    def __init__(self, config: Qwen3_5Config, *, dtype=None, device=None) -> None:
        super().__init__()
        kw = {k: v for k, v in (("dtype", dtype), ("device", device)) if v is not None}
        self.model = Qwen3_5Model(config, dtype=dtype, device=device)
        self.tied = config.text_config.tie_word_embeddings
        if not self.tied:
            self.lm_head = Linear(config.text_config.hidden_size, config.text_config.vocab_size, bias=False, prefix="lm_head", **kw)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, **kw) -> torch.Tensor:
        h = self.model(input_ids, **kw)
        return F.linear(h, self.model.language_model.embed_tokens.weight) if self.tied else self.lm_head(h)


__all__ = ["Qwen3_5GatedDeltaNet", "Qwen3_5Attention", "Qwen3_5DecoderLayer", "Qwen3_5TextModel", "Qwen3_5Model",
           "Qwen3_5ForConditionalGeneration", "RMSNormGated", "ZeroCentredRMS", "qwen3_5_weight_remap"]
