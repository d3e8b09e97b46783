"""Shared attention pieces: enums, mask helpers and the eager fp32-softmax reference.

Reference: phyai/src/phyai/layers/attention/{enums,common,utils}.py.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass

import torch


class AttnMode(enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"
    MIXED = "mixed"


class AttnLayout(enum.Enum):
    PADDED = "padded"      # (B, S, H, D)
    RAGGED = "ragged"      # (T, H, D) + cu_seqlens


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """(..., Hkv, D) -> (..., Hkv * n_rep, D); each KV head serves n_rep consecutive query heads."""
    return x if n_rep == 1 else x.repeat_interleave(n_rep, dim=-2)


def build_padded_mask(seq_lens: torch.Tensor, max_len: int, *, causal: bool = False,
                      sliding_window: int | None = None) -> torch.Tensor:
    """Boolean (B, 1, S, S) mask, True = attend; rows/cols beyond each length are False."""
    B = seq_lens.shape[0]
    ar = torch.arange(max_len, device=seq_lens.device)
    valid = ar[None, :] < seq_lens[:, None]                      # (B, S)
    m = valid[:, None, :, None] & valid[:, None, None, :]
    if causal:
        m = m & (ar[None, None, :, None] >= ar[None, None, None, :])
    if sliding_window is not None:
        m = m & ((ar[None, None, :, None] - ar[None, None, None, :]) < sliding_window)
    return m


def eager_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float | None = None,
               mask: torch.Tensor | None = None, causal: bool = False, logits_soft_cap: float | None = None) -> torch.Tensor:
    """q (B, Sq, Hq, D), k/v (B, Sk, Hkv, D) -> (B, Sq, Hq, D); softmax in fp32."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    kk, vv = repeat_kv(k, Hq // Hkv), repeat_kv(v, Hq // Hkv)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kk.float()) * scale
    if logits_soft_cap:
        s = logits_soft_cap * torch.tanh(s / logits_soft_cap)
    if causal:
        qi = torch.arange(Sq, device=q.device)[:, None] + (Sk - Sq)
        s = s.masked_fill(torch.arange(Sk, device=q.device)[None, :] > qi, float("-inf"))
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.nan_to_num(torch.softmax(s, dim=-1))
    return torch.einsum("bhqk,bkhd->bqhd", p, vv.float()).to(q.dtype)


@dataclass
class RaggedMeta:
    """Ragged batch: sequence b owns tokens [cu[b], cu[b+1])."""

    cu_seqlens: torch.Tensor      # (B+1,) int32
    max_len: int


__all__ = ["AttnMode", "AttnLayout", "repeat_kv", "build_padded_mask", "eager_attn", "RaggedMeta"]
