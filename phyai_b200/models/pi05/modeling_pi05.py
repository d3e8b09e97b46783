"""Pi0.5 model definition: parameters, checkpoint keys and the eager execution path.

The modules here own the weights (with the upstream lerobot / openpi checkpoint key
names, reference: phyai/src/phyai/models/pi05/modeling_pi05.py:140-1184) and an eager
``forward`` built from this package's layers. The eager path runs anywhere (CPU fp32
for tests, CUDA for debugging and tensor dumps) and is the numerical oracle of the
static execution plan in ``plan_pi05.py``, which is what serves requests on B200.

Math summary
* vision: 14x14 patch embed + learned positions, 27 pre-LayerNorm blocks
  (biased q/k/v/out, GELU-tanh MLP), post LayerNorm, linear projector to the LM width;
* prefix LM: token embedding scaled by sqrt(hidden); 18 Gemma blocks, bidirectional
  attention over [image tokens | prompt tokens], 8 query heads on 1 KV head, RoPE,
  (1+w) RMSNorm, GeGLU MLP; only its per-layer K/V matter downstream;
* action expert: 18 blocks over the 50 action tokens, AdaRMSNorm conditioned on the
  flow-matching time, attention over [prefix K/V | own K/V], gated residuals;
* sampler: x <- x + dt * v(x, t), t = 1 - i/N, dt = -1/N, from x ~ N(0, 1).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from ...engine_config import get_engine_config, resolve_engine_defaults
from ...layers.layer_norm import AdaRMSNorm, GemmaRMSNorm, LayerNorm
from ...layers.linear import (ColumnParallelLinear, MergedColumnParallelLinear, QKVParallelLinear,
                              ReplicatedLinear, RowParallelLinear)
from ...layers.rotary_embedding import RotaryEmbedding
from ...ops import ref
from .configuration_pi05 import GemmaExpertConfig, PaliGemmaTextConfig, PI05Config, SiglipVisionConfig

PALIGEMMA = "paligemma_with_expert.paligemma"
EXPERT = "paligemma_with_expert.gemma_expert"


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False) -> torch.Tensor:
    """One sequence: q (T, Hq, D), k/v (S, Hkv, D) -> (T, Hq*D); fp32 softmax."""
    T, S = q.shape[0], k.shape[0]
    z = torch.zeros(1, dtype=torch.int32, device=q.device)
    o = ref.attention(q, k, v, z, z + T, z, z + S, causal=causal)
    return o.reshape(T, -1)


# ------------------------------------------------------------------- vision
class SiglipBlock(nn.Module):
    def __init__(self, cfg: SiglipVisionConfig, dtype, prefix: str, axis: str | None = "tp") -> None:
        super().__init__()
        H, I = cfg.hidden_size, cfg.intermediate_size
        self.num_heads, self.head_dim = cfg.num_attention_heads, cfg.head_dim
        self.ln1 = LayerNorm(H, cfg.layer_norm_eps, dtype=dtype, prefix=f"{prefix}.layer_norm1")
        self.qkv = QKVParallelLinear(H, cfg.head_dim, cfg.num_attention_heads, bias=True, params_dtype=dtype,
                                     prefix=f"{prefix}.self_attn.qkv_proj", axis=axis)
        self.out = RowParallelLinear(H, H, bias=True, params_dtype=dtype, prefix=f"{prefix}.self_attn.out_proj", axis=axis)
        self.ln2 = LayerNorm(H, cfg.layer_norm_eps, dtype=dtype, prefix=f"{prefix}.layer_norm2")
        self.fc1 = ColumnParallelLinear(H, I, bias=True, params_dtype=dtype, prefix=f"{prefix}.mlp.fc1", axis=axis)
        self.fc2 = RowParallelLinear(I, H, bias=True, params_dtype=dtype, prefix=f"{prefix}.mlp.fc2", axis=axis)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """h: (n_img, patches, H)."""
        n, p, _ = h.shape
        x = self.ln1(h)
        qkv, _ = self.qkv(x)
        q, k, v = qkv.split([self.qkv.q_size, self.qkv.kv_size, self.qkv.kv_size], dim=-1)
        outs = []
        for i in range(n):
            outs.append(dense_attention(q[i].reshape(p, -1, self.head_dim), k[i].reshape(p, -1, self.head_dim),
                                        v[i].reshape(p, -1, self.head_dim)))
        a, _ = self.out(torch.stack(outs))
        h = h + a
        m, _ = self.fc1(self.ln2(h))
        m, _ = self.fc2(ref.act_fn(m.float(), "gelu_tanh").to(m.dtype))
        return h + m


class PI05VisionTower(nn.Module):
    """SigLIP-So400m + multi-modal projector; output ``(n_img, patches, text_hidden)``. ``axis``: mesh axis the
    encoder blocks are sharded over; ``None`` keeps the whole tower on every rank (the tensor-parallel plan
    then splits the cameras over the ranks instead of the 72-wide heads and the 4304-wide MLP)."""

    def __init__(self, cfg: SiglipVisionConfig, *, params_dtype=None, prefix: str = f"{PALIGEMMA}.model",
                 axis: str | None = "tp") -> None:
        super().__init__()
        self.axis = axis
        dtype, _, _ = resolve_engine_defaults(params_dtype, None, None)
        dev = get_engine_config().device.target
        self.config, self.compute_dtype = cfg, dtype
        vp = f"{prefix}.vision_tower.vision_model"
        k = cfg.num_channels * cfg.patch_size ** 2
        self.patch_weight = nn.Parameter(torch.empty(cfg.hidden_size, cfg.num_channels, cfg.patch_size, cfg.patch_size,
                                                     dtype=dtype, device=dev), requires_grad=False)
        self.patch_weight.hf_keys = {f"{vp}.embeddings.patch_embedding.weight": None}
        self.patch_bias = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=dtype, device=dev), requires_grad=False)
        self.patch_bias.hf_keys = {f"{vp}.embeddings.patch_embedding.bias": None}
        self.position_embedding = nn.Parameter(torch.zeros(cfg.num_patches, cfg.hidden_size, dtype=dtype, device=dev),
                                               requires_grad=False)
        self.position_embedding.hf_keys = {f"{vp}.embeddings.position_embedding.weight": None}
        self.patch_k = k
        self.blocks = nn.ModuleList([SiglipBlock(cfg, dtype, f"{vp}.encoder.layers.{i}", axis)
                                     for i in range(cfg.num_hidden_layers)])
        self.post_layernorm = LayerNorm(cfg.hidden_size, cfg.layer_norm_eps, dtype=dtype, prefix=f"{vp}.post_layernorm")
        self.projector = ReplicatedLinear(cfg.hidden_size, cfg.projection_dim, bias=True, params_dtype=dtype,
                                          prefix=f"{prefix}.multi_modal_projector.linear")

    def embed_patches(self, pixel_values: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        n = pixel_values.shape[0]
        cols = ref.im2col(pixel_values.to(self.compute_dtype), cfg.patch_size, self.patch_k)
        w = self.patch_weight.reshape(cfg.hidden_size, -1)
        h = (cols.float() @ w.float().t() + self.patch_bias.float()).reshape(n, cfg.num_patches, cfg.hidden_size)
        return (h + self.position_embedding.float()).to(self.compute_dtype)

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """pixel_values: (n_img, C, H, W) already at the tower's resolution."""
        if pixel_values.dim() != 4 or tuple(pixel_values.shape[1:]) != (
                self.config.num_channels, self.config.image_size, self.config.image_size):
            raise ValueError(f"pixel_values {tuple(pixel_values.shape)} does not match "
                             f"(n, {self.config.num_channels}, {self.config.image_size}, {self.config.image_size})")
        h = self.embed_patches(pixel_values)
        for blk in self.blocks:
            h = blk(h)
        h = self.post_layernorm(h)
        y, _ = self.projector(h)
        return y


# ------------------------------------------------------------------ prefix LM
class GemmaMLP(nn.Module):
    def __init__(self, hidden: int, inter: int, dtype, prefix: str, axis: str | None = "tp") -> None:
        super().__init__()
        self.gate_up = MergedColumnParallelLinear(hidden, [inter, inter], bias=False, params_dtype=dtype,
                                                  interleave=True, prefix=f"{prefix}.gate_up_proj", axis=axis)
        self.down = RowParallelLinear(inter, hidden, bias=False, params_dtype=dtype, prefix=f"{prefix}.down_proj", axis=axis)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gu, _ = self.gate_up(x)
        y, _ = self.down(ref.gated_act(gu, "gelu_tanh", interleaved=True))
        return y


class GemmaAttentionProj(nn.Module):
    """q/k/v + o projections of one Gemma block (the attention itself is the caller's)."""

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, dtype, prefix: str, axis: str | None = "tp") -> None:
        super().__init__()
        self.head_dim = head_dim
        self.qkv = QKVParallelLinear(hidden, head_dim, heads, kv_heads, bias=False, params_dtype=dtype,
                                     prefix=f"{prefix}.qkv_proj", axis=axis)
        self.o = RowParallelLinear(heads * head_dim, hidden, bias=False, params_dtype=dtype, prefix=f"{prefix}.o_proj", axis=axis)

    def project_qkv(self, x: torch.Tensor):
        qkv, _ = self.qkv(x)
        q, k, v = qkv.split([self.qkv.q_size, self.qkv.kv_size, self.qkv.kv_size], dim=-1)
        T = x.shape[0]
        return (q.reshape(T, -1, self.head_dim), k.reshape(T, -1, self.head_dim), v.reshape(T, -1, self.head_dim))


class PaliGemmaDecoderLayer(nn.Module):
    def __init__(self, cfg: PaliGemmaTextConfig, dtype, prefix: str) -> None:
        super().__init__()
        self.input_layernorm = GemmaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, prefix=f"{prefix}.input_layernorm")
        self.attn = GemmaAttentionProj(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                       dtype, f"{prefix}.self_attn")
        self.post_attention_layernorm = GemmaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype,
                                                     prefix=f"{prefix}.post_attention_layernorm")
        self.mlp = GemmaMLP(cfg.hidden_size, cfg.intermediate_size, dtype, f"{prefix}.mlp")

    def forward(self, h: torch.Tensor, cos_sin: torch.Tensor):
        """h (T, H) one sequence. Returns (h, k, v) with k/v rotated, ready to cache."""
        q, k, v = self.attn.project_qkv(self.input_layernorm(h))
        q, k = ref.apply_rope(q, cos_sin), ref.apply_rope(k, cos_sin)
        a, _ = self.attn.o(dense_attention(q, k, v))
        h = h + a
        h = h + self.mlp(self.post_attention_layernorm(h))
        return h, k, v


class PaliGemmaLanguageModel(nn.Module):
    def __init__(self, cfg: PaliGemmaTextConfig, *, params_dtype=None, prefix: str = f"{PALIGEMMA}.model.language_model") -> None:
        super().__init__()
        dtype, _, _ = resolve_engine_defaults(params_dtype, None, None)
        dev = get_engine_config().device.target
        self.config = cfg
        self.embed_scale = float(cfg.hidden_size) ** 0.5
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=dev),
                                         requires_grad=False)
        self.embed_tokens.hf_keys = {f"{PALIGEMMA}.lm_head.weight": None}
        self.layers = nn.ModuleList([PaliGemmaDecoderLayer(cfg, dtype, f"{prefix}.layers.{i}")
                                     for i in range(cfg.num_hidden_layers)])
        self.norm = GemmaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, prefix=f"{prefix}.norm")

    def embed_lang(self, input_ids: torch.Tensor) -> torch.Tensor:
        return ref.embedding(input_ids, self.embed_tokens, scale=self.embed_scale)


# ------------------------------------------------------------- action expert
class PI05ExpertLayer(nn.Module):
    def __init__(self, cfg: GemmaExpertConfig, dtype, prefix: str, axis: str | None = "tp") -> None:
        super().__init__()
        self.input_layernorm = AdaRMSNorm(cfg.hidden_size, cfg.adarms_cond_dim, cfg.rms_norm_eps, dtype=dtype,
                                          prefix=f"{prefix}.input_layernorm")
        self.attn = GemmaAttentionProj(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                       dtype, f"{prefix}.self_attn", axis)
        self.post_attention_layernorm = AdaRMSNorm(cfg.hidden_size, cfg.adarms_cond_dim, cfg.rms_norm_eps, dtype=dtype,
                                                   prefix=f"{prefix}.post_attention_layernorm")
        self.mlp = GemmaMLP(cfg.hidden_size, cfg.intermediate_size, dtype, f"{prefix}.mlp", axis)

    def forward(self, h: torch.Tensor, cond: torch.Tensor, cos_sin: torch.Tensor, k_prefix: torch.Tensor,
                v_prefix: torch.Tensor) -> torch.Tensor:
        """h (T, H) one sample's action tokens; cond (1, cond_dim); k/v_prefix (P, Hkv, D)."""
        x, gate = self.input_layernorm(h, cond.expand(h.shape[0], -1))
        q, k, v = self.attn.project_qkv(x)
        q, k = ref.apply_rope(q, cos_sin), ref.apply_rope(k, cos_sin)
        a, _ = self.attn.o(dense_attention(q, torch.cat([k_prefix, k]), torch.cat([v_prefix, v])))
        h = torch.addcmul(h.float(), a.float(), gate.float()).to(h.dtype)
        x, gate = self.post_attention_layernorm(h, cond.expand(h.shape[0], -1))
        return torch.addcmul(h.float(), self.mlp(x).float(), gate.float()).to(h.dtype)


class PI05ExpertStack(nn.Module):
    """The action expert. ``axis``: mesh axis its projections are sharded over; ``None`` keeps the whole expert
    (0.6 GB in bf16) on every rank, so that a tensor-parallel group runs the Euler loop without communication."""

    def __init__(self, cfg: GemmaExpertConfig, *, params_dtype=None, prefix: str = f"{EXPERT}.model", axis: str | None = "tp") -> None:
        super().__init__()
        dtype, _, _ = resolve_engine_defaults(params_dtype, None, None)
        self.config, self.axis = cfg, axis
        self.layers = nn.ModuleList([PI05ExpertLayer(cfg, dtype, f"{prefix}.layers.{i}", axis)
                                     for i in range(cfg.num_hidden_layers)])
        self.norm = AdaRMSNorm(cfg.hidden_size, cfg.adarms_cond_dim, cfg.rms_norm_eps, dtype=dtype, prefix=f"{prefix}.norm")


class ActionTimeHeads(nn.Module):
    def __init__(self, cfg: PI05Config, *, params_dtype=None) -> None:
        super().__init__()
        dtype, _, _ = resolve_engine_defaults(params_dtype, None, None)
        H, A = cfg.expert.hidden_size, cfg.max_action_dim
        self.config = cfg
        self.action_in_proj = ReplicatedLinear(A, H, bias=True, params_dtype=dtype, prefix="action_in_proj")
        self.action_out_proj = ReplicatedLinear(H, A, bias=True, params_dtype=dtype, prefix="action_out_proj")
        self.time_mlp_in = ReplicatedLinear(H, H, bias=True, params_dtype=dtype, prefix="time_mlp_in")
        self.time_mlp_out = ReplicatedLinear(H, H, bias=True, params_dtype=dtype, prefix="time_mlp_out")

    def embed_time(self, t: torch.Tensor) -> torch.Tensor:
        """(B,) times -> (B, H) AdaRMS condition: sinusoid -> Linear -> SiLU -> Linear -> SiLU."""
        cfg = self.config
        emb = ref.sinusoidal_time_embedding(t, cfg.expert.hidden_size, cfg.min_period, cfg.max_period)
        emb = emb.to(self.time_mlp_in.weight.dtype)
        h, _ = self.time_mlp_in(emb)
        h = torch.nn.functional.silu(h.float()).to(h.dtype)
        h, _ = self.time_mlp_out(h)
        return torch.nn.functional.silu(h.float()).to(h.dtype)


class PI05Model(nn.Module):
    def __init__(self, config: PI05Config, *, vision_params_dtype: torch.dtype | None = None,
                 device: str | None = None, params_dtype: torch.dtype | None = None, vision_axis: str | None = "tp",
                 expert_axis: str | None = "tp") -> None:
        super().__init__()
        dtype, _, _ = resolve_engine_defaults(params_dtype, None, None)
        self.config, self.params_dtype = config, dtype
        self.vision = PI05VisionTower(config.vision, params_dtype=vision_params_dtype or dtype, axis=vision_axis)
        self.paligemma_lm = PaliGemmaLanguageModel(config.text, params_dtype=dtype)
        self.expert_stack = PI05ExpertStack(config.expert, params_dtype=dtype, axis=expert_axis)
        self.heads = ActionTimeHeads(config, params_dtype=dtype)
        self.rope = RotaryEmbedding(config.text.head_dim, config.text.max_position_embeddings, config.text.rope_theta,
                                    device=get_engine_config().device.target)

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> "PI05Model":
        """Deterministic random weights (norm scales stay at identity); used by benchmarks and tests."""
        g = torch.Generator().manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() == 1 and ("norm" in name and "dense" not in name) and "bias" not in name:
                continue
            if "layernorm.weight" in name or name.endswith("ln1.weight") or name.endswith("ln2.weight"):
                continue
            scale = 0.3 if "position_embedding" in name else std
            if name.endswith("embed_tokens"):
                scale = 1.0 / math.sqrt(p.shape[1])
            p.copy_((torch.randn(p.shape, generator=g) * scale).to(p.dtype))
        return self

    # --------------------------------------------------------------- oracle
    @torch.no_grad()
    def encode_prefix(self, pixel_values: torch.Tensor, input_ids: torch.Tensor, lang_len: int):
        """One robot: pixel_values (n_img, C, H, W), input_ids (L,). Returns (per-layer [(k, v)], prefix_len)."""
        img = self.vision(pixel_values).reshape(-1, self.config.text.hidden_size).to(self.params_dtype)
        lang = self.paligemma_lm.embed_lang(input_ids[:lang_len]).to(self.params_dtype)
        h = torch.cat([img, lang], dim=0)
        P = h.shape[0]
        cs = self.rope.cos_sin_cache[:P]
        kv = []
        for layer in self.paligemma_lm.layers:
            h, k, v = layer(h, cs)
            kv.append((k, v))
        return kv, P

    @torch.no_grad()
    def denoise(self, kv, prefix_len: int, noise: torch.Tensor) -> torch.Tensor:
        """One robot: noise (chunk, action_dim) -> action chunk after the Euler loop (fp32 state)."""
        cfg = self.config
        N = cfg.num_inference_steps
        dt = -1.0 / N
        x = noise.float().clone()
        cs = self.rope.cos_sin_cache[prefix_len:prefix_len + cfg.chunk_size]
        for i in range(N):
            t = torch.full((1,), 1.0 + i * dt, dtype=torch.float32, device=x.device)
            cond = self.heads.embed_time(t)
            h, _ = self.heads.action_in_proj(x.to(self.params_dtype))
            for layer, (kp, vp) in zip(self.expert_stack.layers, kv):
                h = layer(h, cond, cs, kp, vp)
            h, _ = self.expert_stack.norm(h, cond.expand(h.shape[0], -1))
            v_t, _ = self.heads.action_out_proj(h)
            x = x + dt * v_t.float()
        return x

    @torch.no_grad()
    def sample_actions(self, pixel_values: torch.Tensor, input_ids: torch.Tensor, lang_lens: torch.Tensor,
                       noise: torch.Tensor) -> torch.Tensor:
        """Batch eager path. pixel_values (B, n_img, C, H, W); returns (B, chunk, action_dim) fp32."""
        outs = []
        for b in range(pixel_values.shape[0]):
            kv, P = self.encode_prefix(pixel_values[b], input_ids[b], int(lang_lens[b]))
            outs.append(self.denoise(kv, P, noise[b]))
        return torch.stack(outs)


__all__ = ["PI05Model", "PI05VisionTower", "PaliGemmaLanguageModel", "PI05ExpertStack", "ActionTimeHeads",
           "PaliGemmaDecoderLayer", "PI05ExpertLayer", "GemmaMLP", "GemmaAttentionProj", "SiglipBlock",
           "dense_attention"]
