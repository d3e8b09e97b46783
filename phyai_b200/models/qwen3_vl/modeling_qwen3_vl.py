"""Qwen3-VL: a reference implementation (prefill only, not registered as a serving plugin).

Vision tower: Conv3d-equivalent patch embedding (a linear over flattened t x p x p patches), learned
position table interpolated bilinearly to each image's grid, 2-D rotary attention that is block
diagonal over the images of a batch (ragged: one packed sequence, ``cu_seqlens`` marks the
images), a 2x2 patch merger, and DeepStack: the merged features of some intermediate blocks are
added to the hidden states of the first text layers at the image positions. Text: a Qwen3 decoder
(qk-norm, GQA, SwiGLU) with three-axis interleaved mRoPE.

Parameter names follow the public checkpoints (``model.visual.*``, ``model.language_model.*``,
``lm_head``). Reference: phyai/src/phyai/models/qwen3_vl/modeling_qwen3_vl.py:32-1045.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...layers.rotary_embedding import MRotaryEmbedding, rotate_half
from .configuration_qwen3_vl import Qwen3VLConfig, Qwen3VLTextConfig, Qwen3VLVisionConfig


def _key(p: nn.Parameter, name: str) -> nn.Parameter:
    p.hf_keys = {name: None}
    p.requires_grad_(False)
    return p


class Linear(nn.Linear):
    """``nn.Linear`` whose parameters know their checkpoint keys."""

    def __init__(self, i: int, o: int, *, bias: bool = True, prefix: str, dtype=None, device=None) -> None:
        super().__init__(i, o, bias=bias, dtype=dtype, device=device)
        _key(self.weight, f"{prefix}.weight")
        if bias:
            _key(self.bias, f"{prefix}.bias")


class RMS(nn.Module):
    def __init__(self, d: int, eps: float, prefix: str, dtype=None, device=None) -> None:
        super().__init__()
        self.eps = eps
        self.weight = _key(nn.Parameter(torch.ones(d, dtype=dtype, device=device)), f"{prefix}.weight")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


# ---------------------------------------------------------------- vision helpers
def get_vision_cu_seqlens(grid_thw: torch.Tensor) -> torch.Tensor:
    """(n, 3) grids -> cumulative patch counts with one entry per FRAME (attention never crosses frames)."""
    per_frame = torch.repeat_interleave(grid_thw[:, 1] * grid_thw[:, 2], grid_thw[:, 0])
    return F.pad(per_frame.cumsum(0), (1, 0)).to(torch.int32)


def get_vision_position_ids(grid_thw: torch.Tensor, merge: int) -> torch.Tensor:
    """(total_patches, 2) row / column of every patch, in the merge-block-major order the patches are packed in."""
    out = []
    for t, h, w in grid_thw.tolist():
        hh = torch.arange(h)[:, None].expand(h, w).reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).reshape(-1)
        ww = torch.arange(w)[None, :].expand(h, w).reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).reshape(-1)
        out.append(torch.stack([hh, ww], -1).repeat(t, 1))
    return torch.cat(out)


def get_vision_bilinear_indices_and_weights(grid_thw: torch.Tensor, side: int, merge: int):
    """For each patch: the 4 entries of the (side x side) position table around its fractional location, and their weights."""
    idx, wgt = [], []
    for t, h, w in grid_thw.tolist():
        ys, xs = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
        y0, x0 = ys.floor().long(), xs.floor().long()
        y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
        fy, fx = (ys - y0)[:, None], (xs - x0)[None, :]
        i4 = torch.stack([y0[:, None] * side + x0[None], y0[:, None] * side + x1[None], y1[:, None] * side + x0[None], y1[:, None] * side + x1[None]], 0)
        w4 = torch.stack([(1 - fy) * (1 - fx), (1 - fy) * fx, fy * (1 - fx), fy * fx], 0)
        order = lambda a: a.reshape(4, h // merge, merge, w // merge, merge).permute(0, 1, 3, 2, 4).reshape(4, -1)  # noqa: E731
        idx.append(order(i4).repeat(1, t))
        wgt.append(order(w4).repeat(1, t))
    return torch.cat(idx, 1), torch.cat(wgt, 1)


def apply_rotary_pos_emb_vision(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    cos, sin = cos[:, None].float(), sin[:, None].float()
    return ((q.float() * cos + rotate_half(q.float()) * sin).to(q.dtype), (k.float() * cos + rotate_half(k.float()) * sin).to(k.dtype))


def ragged_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu: torch.Tensor) -> torch.Tensor:
    """(S, H, D) packed; attention inside each [cu[i], cu[i+1]) segment only."""
    out = torch.empty_like(q)
    bounds = cu.tolist()
    for a, b in zip(bounds[:-1], bounds[1:]):
        o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None], v[a:b].transpose(0, 1)[None])
        out[a:b] = o[0].transpose(0, 1)
    return out


class VisionBlock(nn.Module):
    def __init__(self, c: Qwen3VLVisionConfig, prefix: str, **kw) -> None:
        super().__init__()
        self.heads = c.num_heads
        self.norm1 = nn.LayerNorm(c.hidden_size, eps=1e-6, **kw)
        self.norm2 = nn.LayerNorm(c.hidden_size, eps=1e-6, **kw)
        for n in ("norm1", "norm2"):
            _key(getattr(self, n).weight, f"{prefix}.{n}.weight"), _key(getattr(self, n).bias, f"{prefix}.{n}.bias")
        self.qkv = Linear(c.hidden_size, 3 * c.hidden_size, prefix=f"{prefix}.attn.qkv", **kw)
        self.proj = Linear(c.hidden_size, c.hidden_size, prefix=f"{prefix}.attn.proj", **kw)
        self.fc1 = Linear(c.hidden_size, c.intermediate_size, prefix=f"{prefix}.mlp.linear_fc1", **kw)
        self.fc2 = Linear(c.intermediate_size, c.hidden_size, prefix=f"{prefix}.mlp.linear_fc2", **kw)

    def forward(self, x: torch.Tensor, cu: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        S, C = x.shape
        q, k, v = self.qkv(self.norm1(x)).reshape(S, 3, self.heads, C // self.heads).unbind(1)
        q, k = apply_rotary_pos_emb_vision(q, k, cos, sin)
        x = x + self.proj(ragged_attention(q, k, v, cu).reshape(S, C))
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x)), approximate="tanh"))


class PatchMerger(nn.Module):
    """merge x merge neighbouring patches -> one token of the text width. ``postshuffle``: norm after the concatenation (DeepStack taps)."""

    def __init__(self, c: Qwen3VLVisionConfig, prefix: str, postshuffle: bool, **kw) -> None:
        super().__init__()
        self.group = c.spatial_merge_size ** 2
        d = c.hidden_size * self.group
        self.postshuffle = postshuffle
        self.norm = nn.LayerNorm(d if postshuffle else c.hidden_size, eps=1e-6, **kw)
        _key(self.norm.weight, f"{prefix}.norm.weight"), _key(self.norm.bias, f"{prefix}.norm.bias")
        self.fc1 = Linear(d, d, prefix=f"{prefix}.linear_fc1", **kw)
        self.fc2 = Linear(d, c.out_hidden_size, prefix=f"{prefix}.linear_fc2", **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.norm(x.reshape(-1, self.norm.normalized_shape[0])) if self.postshuffle else self.norm(x)
        return self.fc2(F.gelu(self.fc1(x.reshape(-1, self.fc1.in_features))))


class Qwen3VLVisionModel(nn.Module):
    def __init__(self, c: Qwen3VLVisionConfig, prefix: str = "model.visual", **kw) -> None:
        super().__init__()
        self.c = c
        self.patch_embed = Linear(c.in_channels * c.temporal_patch_size * c.patch_size ** 2, c.hidden_size, prefix=f"{prefix}.patch_embed.proj", **kw)
        self.patch_embed.weight.weight_loader = lambda p, t, sid=None: p.data.copy_(t.reshape(p.shape).to(p.dtype))   # checkpoint: Conv3d kernel
        self.pos_embed = _key(nn.Parameter(torch.zeros(c.num_position_embeddings, c.hidden_size, **kw)), f"{prefix}.pos_embed.weight")
        self.blocks = nn.ModuleList([VisionBlock(c, f"{prefix}.blocks.{i}", **kw) for i in range(c.depth)])
        self.merger = PatchMerger(c, f"{prefix}.merger", False, **kw)
        self.deepstack_merger_list = nn.ModuleList([PatchMerger(c, f"{prefix}.deepstack_merger_list.{i}", True, **kw)
                                                    for i in range(len(c.deepstack_visual_indexes))])
        hd = c.hidden_size // c.num_heads
        self.register_buffer("inv_freq", 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2).float() / (hd // 2))), persistent=False)

    def forward(self, patches: torch.Tensor, grid_thw: torch.Tensor):
        """``patches`` (total_patches, C * t * p * p) packed over all images -> (merged tokens (n, out), [DeepStack features])."""
        c = self.c
        x = self.patch_embed(patches)
        side = int(c.num_position_embeddings ** 0.5)
        idx, wgt = get_vision_bilinear_indices_and_weights(grid_thw, side, c.spatial_merge_size)
        x = x + (self.pos_embed[idx.to(x.device)] * wgt.to(x.device, x.dtype)[..., None]).sum(0)
        pos = get_vision_position_ids(grid_thw, c.spatial_merge_size).to(x.device)
        ang = pos[:, :, None].float() * self.inv_freq[None, None].to(x.device)          # (S, 2, hd/4)
        emb = ang.flatten(1).repeat(1, 2)
        cos, sin = emb.cos(), emb.sin()
        cu = get_vision_cu_seqlens(grid_thw)
        taps = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cu, cos, sin)
            if i in c.deepstack_visual_indexes:
                taps.append(self.deepstack_merger_list[c.deepstack_visual_indexes.index(i)](x))
        return self.merger(x), taps


# ---------------------------------------------------------------- text
class TextLayer(nn.Module):
    def __init__(self, c: Qwen3VLTextConfig, prefix: str, **kw) -> None:
        super().__init__()
        self.c = c
        H, D, nq, nk = c.hidden_size, c.head_dim, c.num_attention_heads, c.num_key_value_heads
        p = f"{prefix}.self_attn"
        self.q_proj, self.k_proj = Linear(H, nq * D, bias=False, prefix=f"{p}.q_proj", **kw), Linear(H, nk * D, bias=False, prefix=f"{p}.k_proj", **kw)
        self.v_proj, self.o_proj = Linear(H, nk * D, bias=False, prefix=f"{p}.v_proj", **kw), Linear(nq * D, H, bias=False, prefix=f"{p}.o_proj", **kw)
        self.q_norm, self.k_norm = RMS(D, c.rms_norm_eps, f"{p}.q_norm", **kw), RMS(D, c.rms_norm_eps, f"{p}.k_norm", **kw)
        self.input_layernorm = RMS(H, c.rms_norm_eps, f"{prefix}.input_layernorm", **kw)
        self.post_attention_layernorm = RMS(H, c.rms_norm_eps, f"{prefix}.post_attention_layernorm", **kw)
        m = f"{prefix}.mlp"
        self.gate_proj, self.up_proj = Linear(H, c.intermediate_size, bias=False, prefix=f"{m}.gate_proj", **kw), Linear(H, c.intermediate_size, bias=False, prefix=f"{m}.up_proj", **kw)
        self.down_proj = Linear(c.intermediate_size, H, bias=False, prefix=f"{m}.down_proj", **kw)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, mask: torch.Tensor | None) -> torch.Tensor:
        B, S, _ = x.shape
        c = self.c
        h = self.input_layernorm(x)
        q = self.q_norm(self.q_proj(h).reshape(B, S, c.num_attention_heads, c.head_dim)).transpose(1, 2)
        k = self.k_norm(self.k_proj(h).reshape(B, S, c.num_key_value_heads, c.head_dim)).transpose(1, 2)
        v = self.v_proj(h).reshape(B, S, c.num_key_value_heads, c.head_dim).transpose(1, 2)
        cs, sn = cos[:, None].float(), sin[:, None].float()
        q = (q.float() * cs + rotate_half(q.float()) * sn).to(q.dtype)
        k = (k.float() * cs + rotate_half(k.float()) * sn).to(k.dtype)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=mask is None, enable_gqa=True)
        x = x + self.o_proj(o.transpose(1, 2).reshape(B, S, -1))
        h = self.post_attention_layernorm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class Qwen3VLTextModel(nn.Module):
    def __init__(self, c: Qwen3VLTextConfig, prefix: str = "model.language_model", **kw) -> None:
        super().__init__()
        self.c = c
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size, **kw)
        _key(self.embed_tokens.weight, f"{prefix}.embed_tokens.weight")
        self.layers = nn.ModuleList([TextLayer(c, f"{prefix}.layers.{i}", **kw) for i in range(c.num_hidden_layers)])
        self.norm = RMS(c.hidden_size, c.rms_norm_eps, f"{prefix}.norm", **kw)
        self.rotary = MRotaryEmbedding(c.head_dim, c.mrope_section, c.rope_theta, interleaved=True)

    def forward(self, inputs_embeds: torch.Tensor, position_ids: torch.Tensor, *, attention_mask: torch.Tensor | None = None,
                deepstack: list[torch.Tensor] | None = None, visual_pos: torch.Tensor | None = None) -> torch.Tensor:
        """``position_ids`` (3, B, S). ``deepstack[i]`` is added to the output of layer ``i`` at ``visual_pos`` (B, S) bool."""
        B, S, _ = inputs_embeds.shape
        cs = torch.stack([self.rotary.cos_sin(position_ids[:, b].float()) for b in range(B)])     # (B, S, head_dim)
        half = self.c.head_dim // 2
        cos, sin = cs[..., :half].repeat(1, 1, 2), cs[..., half:].repeat(1, 1, 2)
        mask = None
        if attention_mask is not None:
            causal = torch.ones(S, S, dtype=torch.bool, device=inputs_embeds.device).tril()
            mask = causal[None, None] & attention_mask[:, None, None].bool()
        x = inputs_embeds
        for i, layer in enumerate(self.layers):
            x = layer(x, cos, sin, mask)
            if deepstack is not None and i < len(deepstack):
                x = x.clone()
                x[visual_pos] = x[visual_pos] + deepstack[i].to(x.dtype)
        return self.norm(x)


class Qwen3VLModel(nn.Module):
    def __init__(self, config: Qwen3VLConfig, *, dtype=None, device=None) -> None:
        super().__init__()
        kw = {k: v for k, v in (("dtype", dtype), ("device", device)) if v is not None}
        self.config = config
        self.visual = Qwen3VLVisionModel(config.vision_config, **kw)
        self.language_model = Qwen3VLTextModel(config.text_config, **kw)

    def get_rope_index(self, input_ids: torch.Tensor, grid_thw: torch.Tensor | None) -> torch.Tensor:
        """(3, B, S) positions: text tokens advance all three axes together; an image's tokens share the temporal
        index and spread over (row, column) of its merged grid; text after an image resumes past its largest index."""
        B, S = input_ids.shape
        m = self.config.vision_config.spatial_merge_size
        pos = torch.zeros(3, B, S, dtype=torch.long)
        grids = [] if grid_thw is None else grid_thw.tolist()
        gi = 0
        for b in range(B):
            ids = input_ids[b].tolist()
            s, nxt = 0, 0
            while s < S:
                if ids[s] in (self.config.image_token_id, self.config.video_token_id) and gi < len(grids):
                    t, h, w = grids[gi]
                    gi += 1
                    hh, ww = h // m, w // m
                    n = t * hh * ww
                    tt = torch.arange(t).repeat_interleave(hh * ww)
                    pos[0, b, s:s + n] = nxt + tt
                    pos[1, b, s:s + n] = nxt + torch.arange(hh).repeat_interleave(ww).repeat(t)
                    pos[2, b, s:s + n] = nxt + torch.arange(ww).repeat(hh * t)
                    nxt += max(t, hh, ww)
                    s += n
                else:
                    pos[:, b, s] = nxt
                    nxt += 1
                    s += 1
        return pos.to(input_ids.device)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, *, pixel_patches: torch.Tensor | None = None, grid_thw: torch.Tensor | None = None,
                attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        x = self.language_model.embed_tokens(input_ids)
        deep, vis_pos = None, None
        if pixel_patches is not None:
            feats, deep = self.visual(pixel_patches.to(x.dtype), grid_thw)
            vis_pos = (input_ids == self.config.image_token_id) | (input_ids == self.config.video_token_id)
            if int(vis_pos.sum()) != feats.shape[0]:
                raise ValueError(f"{int(vis_pos.sum())} image placeholder tokens for {feats.shape[0]} visual features")
            x = x.clone()
            x[vis_pos] = feats.to(x.dtype)
        pos = self.get_rope_index(input_ids, grid_thw)
        return self.language_model(x, pos, attention_mask=attention_mask, deepstack=deep, visual_pos=vis_pos)


class Qwen3VLForConditionalGeneration(nn.Module):
    def __init__(self, config: Qwen3VLConfig, *, dtype=None, device=None) -> None:
        super().__init__()
        kw = {k: v for k, v in (("dtype", dtype), ("device", device)) if v is not None}
        self.model = Qwen3VLModel(config, dtype=dtype, device=device)
        self.lm_head = Linear(config.text_config.hidden_size, config.text_config.vocab_size, bias=False, prefix="lm_head", **kw)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, **kw) -> torch.Tensor:
        return self.lm_head(self.model(input_ids, **kw))


__all__ = ["Qwen3VLVisionModel", "Qwen3VLTextModel", "Qwen3VLModel", "Qwen3VLForConditionalGeneration", "get_vision_cu_seqlens",
           "get_vision_position_ids", "get_vision_bilinear_indices_and_weights", "apply_rotary_pos_emb_vision", "ragged_attention"]
