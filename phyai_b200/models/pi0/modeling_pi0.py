"""Pi0 model: parameters, checkpoint keys and the eager path.

Differences from Pi0.5 (reference: phyai/src/phyai/models/pi0/modeling_pi0.py:99-1073):
the suffix is ``[state token | 50 action tokens]``; the state token sees the prefix and
itself, action tokens see prefix + state + all actions; the expert uses Gemma RMSNorm and
plain residuals; the flow time is concatenated to the action embedding and mixed by
``action_time_mlp_in (2H -> H) -> SiLU -> action_time_mlp_out``.

The state token's path never depends on the noisy actions, so its per-layer K/V are
computed once per request and reused by all Euler steps (the reference recomputes them
every step, phyai/src/phyai/models/pi0/model_runner_pi0.py:510-554).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...engine_config import get_engine_config, resolve_engine_defaults
from ...layers.layer_norm import GemmaRMSNorm
from ...layers.linear import ReplicatedLinear
from ...layers.rotary_embedding import RotaryEmbedding
from ...ops import ref
from ..pi05.modeling_pi05 import (EXPERT, PaliGemmaDecoderLayer, PaliGemmaLanguageModel, PI05VisionTower,
                                  dense_attention)
from .configuration_pi0 import PI0Config


class PI0ExpertStack(nn.Module):
    def __init__(self, cfg, *, params_dtype=None, prefix: str = f"{EXPERT}.model") -> None:
        super().__init__()
        dtype, _, _ = resolve_engine_defaults(params_dtype, None, None)
        self.config = cfg
        self.layers = nn.ModuleList([PaliGemmaDecoderLayer(cfg, dtype, f"{prefix}.layers.{i}")
                                     for i in range(cfg.num_hidden_layers)])
        self.norm = GemmaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, prefix=f"{prefix}.norm")


class PI0Heads(nn.Module):
    def __init__(self, cfg: PI0Config, *, params_dtype=None) -> None:
        super().__init__()
        dtype, _, _ = resolve_engine_defaults(params_dtype, None, None)
        H = cfg.expert.hidden_size
        self.config = cfg
        kw = dict(bias=True, params_dtype=dtype)
        self.state_proj = ReplicatedLinear(cfg.max_state_dim, H, prefix="state_proj", **kw)
        self.action_in_proj = ReplicatedLinear(cfg.max_action_dim, H, prefix="action_in_proj", **kw)
        self.action_out_proj = ReplicatedLinear(H, cfg.max_action_dim, prefix="action_out_proj", **kw)
        self.action_time_mlp_in = ReplicatedLinear(2 * H, H, prefix="action_time_mlp_in", **kw)
        self.action_time_mlp_out = ReplicatedLinear(H, H, prefix="action_time_mlp_out", **kw)

    def time_embedding(self, t: torch.Tensor) -> torch.Tensor:
        c = self.config
        return ref.sinusoidal_time_embedding(t, c.expert.hidden_size, c.min_period, c.max_period)

    def embed_action_time(self, x_t: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        """x_t (T, A), t (1,) -> (T, H)."""
        a, _ = self.action_in_proj(x_t.to(self.action_in_proj.weight.dtype))
        te = self.time_embedding(t).to(a.dtype).expand(a.shape[0], -1)
        h, _ = self.action_time_mlp_in(torch.cat([a, te], dim=-1))
        h, _ = self.action_time_mlp_out(F.silu(h.float()).to(h.dtype))
        return h


class PI0Model(nn.Module):
    def __init__(self, config: PI0Config, *, vision_params_dtype: torch.dtype | None = None, device=None,
                 params_dtype: torch.dtype | None = None) -> None:
        super().__init__()
        dtype, _, _ = resolve_engine_defaults(params_dtype, None, None)
        self.config, self.params_dtype = config, dtype
        self.vision = PI05VisionTower(config.vision, params_dtype=vision_params_dtype or dtype)
        self.paligemma_lm = PaliGemmaLanguageModel(config.text, params_dtype=dtype)
        self.expert_stack = PI0ExpertStack(config.expert, params_dtype=dtype)
        self.heads = PI0Heads(config, params_dtype=dtype)
        self.rope = RotaryEmbedding(config.text.head_dim, config.text.max_position_embeddings, config.text.rope_theta,
                                    device=get_engine_config().device.target)

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> "PI0Model":
        g = torch.Generator().manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() == 1 and "norm" in name and "bias" not in name:
                continue
            if name.endswith("ln1.weight") or name.endswith("ln2.weight") or "layernorm.weight" in name:
                continue
            scale = 0.3 if "position_embedding" in name else std
            if name.endswith("embed_tokens"):
                scale = 1.0 / math.sqrt(p.shape[1])
            p.copy_((torch.randn(p.shape, generator=g) * scale).to(p.dtype))
        return self

    # ----------------------------------------------------------------- eager
    @torch.no_grad()
    def encode_prefix(self, pixel_values, input_ids, lang_len: int):
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

    def _expert_layer(self, layer, h, cs, k_ctx, v_ctx):
        """One expert block over rows ``h`` attending [k_ctx | own]. Returns (h, k_own, v_own)."""
        q, k, v = layer.attn.project_qkv(layer.input_layernorm(h))
        q, k = ref.apply_rope(q, cs), ref.apply_rope(k, cs)
        a, _ = layer.attn.o(dense_attention(q, torch.cat([k_ctx, k]), torch.cat([v_ctx, v])))
        h = h + a
        h = h + layer.mlp(layer.post_attention_layernorm(h))
        return h, k, v

    @torch.no_grad()
    def denoise(self, kv, prefix_len: int, state: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        N, dt = cfg.num_inference_steps, -1.0 / cfg.num_inference_steps
        # state token: position prefix_len, sees prefix + itself; computed once
        hs, _ = self.heads.state_proj(state[None].to(self.params_dtype))
        cs_s = self.rope.cos_sin_cache[prefix_len:prefix_len + 1]
        ctx = []
        for layer, (kp, vp) in zip(self.expert_stack.layers, kv):
            hs, ks, vs = self._expert_layer(layer, hs, cs_s, kp, vp)
            ctx.append((torch.cat([kp, ks]), torch.cat([vp, vs])))
        cs_a = self.rope.cos_sin_cache[prefix_len + 1:prefix_len + 1 + cfg.chunk_size]
        x = noise.float().clone()
        for i in range(N):
            t = torch.full((1,), 1.0 + i * dt, dtype=torch.float32, device=x.device)
            h = self.heads.embed_action_time(x.to(self.params_dtype), t)
            for layer, (kc, vc) in zip(self.expert_stack.layers, ctx):
                h, _, _ = self._expert_layer(layer, h, cs_a, kc, vc)
            v_t, _ = self.heads.action_out_proj(self.expert_stack.norm(h))
            x = x + dt * v_t.float()
        return x

    @torch.no_grad()
    def sample_actions(self, pixel_values, input_ids, lang_lens, state, noise) -> torch.Tensor:
        outs = []
        for b in range(pixel_values.shape[0]):
            kv, P = self.encode_prefix(pixel_values[b], input_ids[b], int(lang_lens[b]))
            outs.append(self.denoise(kv, P, state[b], noise[b]))
        return torch.stack(outs)


__all__ = ["PI0Model", "PI0ExpertStack", "PI0Heads"]
