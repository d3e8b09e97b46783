"""Rotary position embeddings.

``RotaryEmbedding`` keeps an fp32 ``cos | sin`` cache and applies rotate-half RoPE
(default / linear / llama3 frequency scaling, partial rotary). ``MRotaryEmbedding``
weaves three position axes (t, h, w) over the frequency bands the way Qwen3-VL
does. Reference: phyai/src/phyai/layers/rotary_embedding.py:97-799.
"""

from __future__ import annotations

import math
from typing import Sequence

import torch
import torch.nn as nn


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def apply_rotary_pos_emb(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """HF convention: ``cos``/``sin`` are (..., D) with the half-table repeated twice."""
    qf, kf = q.float(), k.float()
    return ((qf * cos + rotate_half(qf) * sin).to(q.dtype), (kf * cos + rotate_half(kf) * sin).to(k.dtype))


def compute_inv_freq(rot_dim: int, theta: float, scaling: dict | None = None, device=None) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
    if not scaling:
        return inv
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind in ("default", None):
        return inv
    if kind == "linear":
        return inv / float(scaling["factor"])
    if kind == "llama3":
        factor, lo, hi = float(scaling["factor"]), float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - lo) / (hi - lo)
        mid = (1 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > old / lo, inv / factor, inv)
        is_mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        return torch.where(is_mid, mid, out)
    raise ValueError(f"unknown rope scaling {kind!r}")


def compute_cos_sin_from_inv_freq(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """(P,) positions -> (P, rot_dim) fp32 ``cos(half) | sin(half)``."""
    ang = positions.float()[..., None] * inv_freq.float()
    return torch.cat([ang.cos(), ang.sin()], dim=-1)


class RotaryEmbedding(nn.Module):
    def __init__(self, head_dim: int, max_position: int = 8192, theta: float = 10000.0, *, rotary_dim: int | None = None,
                 scaling: dict | None = None, device=None, max_position_embeddings: int | None = None, rope_theta: float | None = None,
                 rope_type: str = "default", rope_scaling: dict | None = None, partial_rotary_factor: float | None = None,
                 interleave: bool = False, backend: str | None = None) -> None:
        """The keyword spellings of the reference (``max_position_embeddings``, ``rope_theta``, ``rope_type`` +
        ``rope_scaling``, ``partial_rotary_factor``; phyai/src/phyai/layers/rotary_embedding.py:386-398) are taken as
        well; ``backend`` is accepted and ignored (one implementation here); the pairwise-interleaved layout is not built."""
        super().__init__()
        if interleave:
            raise NotImplementedError("RotaryEmbedding rotates halves (the layout of every model here); interleave=True is not built")
        max_position = max_position if max_position_embeddings is None else int(max_position_embeddings)
        theta = theta if rope_theta is None else float(rope_theta)
        if rope_scaling is not None or rope_type != "default":
            scaling = {**(rope_scaling or {}), "rope_type": (rope_scaling or {}).get("rope_type", rope_type)}
        if partial_rotary_factor is not None:
            if not 0.0 < partial_rotary_factor <= 1.0:
                raise ValueError(f"partial_rotary_factor must be in (0, 1], got {partial_rotary_factor}")
            rotary_dim = int(head_dim * partial_rotary_factor)
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim or head_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and <= head_dim={head_dim}")
        self.max_position, self.theta = max_position, theta
        inv = compute_inv_freq(self.rotary_dim, theta, scaling, device)
        table = compute_cos_sin_from_inv_freq(torch.arange(max_position, device=device), inv)
        self.register_buffer("cos_sin_cache", table, persistent=False)

    def get_cos_sin(self, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``(cos, sin)`` for ``positions`` (any shape), each ``(*positions.shape, rotary_dim)`` fp32 with the half-width
        table repeated (the rotate-half layout). Hoist this out of a layer loop when all layers share the positions."""
        cs = self.cos_sin_cache[positions.long()]
        half = cs.shape[-1] // 2
        return torch.cat([cs[..., :half], cs[..., :half]], -1), torch.cat([cs[..., half:], cs[..., half:]], -1)

    def forward(self, positions: torch.Tensor, q: torch.Tensor, k: torch.Tensor):
        """q (T, Hq, D), k (T, Hkv, D), positions (T,). Returns rotated copies."""
        from ..ops import ref

        cs = self.cos_sin_cache[positions.long()]
        return ref.apply_rope(q, cs), ref.apply_rope(k, cs)


class MRotaryEmbedding(nn.Module):
    """Three-axis RoPE: frequency band ``i`` takes its angle from axis ``section_of(i)``.

    ``interleaved=True`` assigns bands round-robin (t, h, w, t, h, w, ...) inside the
    span covered by all sections (Qwen3-VL); otherwise bands are contiguous blocks.
    """

    def __init__(self, head_dim: int, sections: Sequence[int], theta: float = 5e6, *, interleaved: bool = True) -> None:
        super().__init__()
        if sum(sections) != head_dim // 2:
            raise ValueError(f"mrope sections {tuple(sections)} must sum to head_dim/2 = {head_dim // 2}")
        self.head_dim, self.sections, self.theta, self.interleaved = head_dim, tuple(sections), theta, interleaved
        self.register_buffer("inv_freq", compute_inv_freq(head_dim, theta), persistent=False)
        half = head_dim // 2
        axis = torch.zeros(half, dtype=torch.long)
        if interleaved:
            # axis a owns bands a, a+3, a+6, ... until its quota is used; leftovers go to axis 0
            quota = list(self.sections)
            for i in range(half):
                a = i % 3
                if quota[a] > 0:
                    axis[i] = a
                    quota[a] -= 1
                else:
                    axis[i] = 0
                    quota[0] -= 1
        else:
            o = 0
            for a, n in enumerate(self.sections):
                axis[o:o + n] = a
                o += n
        self.register_buffer("band_axis", axis, persistent=False)

    def get_cos_sin(self, position_ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``(cos, sin)`` of shape ``(B, S, head_dim)`` (half-width table repeated) for ``position_ids`` ``(3, B, S)``, or
        ``(B, S)`` read as the same index on all three axes."""
        if position_ids.dim() == 2:
            position_ids = position_ids[None].expand(3, *position_ids.shape)
        if position_ids.dim() != 3 or position_ids.shape[0] != 3:
            raise ValueError(f"position ids are (3, B, S) or (B, S), got {tuple(position_ids.shape)}")
        _, B, S = position_ids.shape
        cs = self.cos_sin(position_ids.reshape(3, B * S)).reshape(B, S, -1)
        half = cs.shape[-1] // 2
        return torch.cat([cs[..., :half], cs[..., :half]], -1), torch.cat([cs[..., half:], cs[..., half:]], -1)

    def cos_sin(self, positions: torch.Tensor) -> torch.Tensor:
        """positions (3, T) float -> (T, head_dim) fp32 ``cos | sin``."""
        dev = positions.device   # the tables are tiny: follow the positions rather than the module
        ang_all = positions.float()[:, :, None] * self.inv_freq.float().to(dev)[None, None, :]   # (3, T, half)
        ang = torch.gather(ang_all, 0, self.band_axis.to(dev)[None, None, :].expand(1, ang_all.shape[1], -1))[0]
        return torch.cat([ang.cos(), ang.sin()], dim=-1)


InterleavedMRotaryEmbedding = MRotaryEmbedding

__all__ = ["rotate_half", "apply_rotary_pos_emb", "compute_inv_freq", "compute_cos_sin_from_inv_freq",
           "RotaryEmbedding", "MRotaryEmbedding", "InterleavedMRotaryEmbedding"]
