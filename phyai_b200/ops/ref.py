"""Plain PyTorch fp32 restatements of every kernel in ``phyai_b200.ops``.

These run anywhere (CPU included). They are the numerical oracle for the CUDA
kernels and the building blocks of the CPU execution path of the models.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def act_fn(x: torch.Tensor, act: str | None) -> torch.Tensor:
    if act in (None, "none"):
        return x
    if act in ("gelu_tanh", "gelu_pytorch_tanh"):
        return F.gelu(x, approximate="tanh")
    if act in ("silu", "swish"):
        return F.silu(x)
    if act in ("gelu", "gelu_erf"):
        return F.gelu(x)
    raise ValueError(f"unknown activation {act!r}")


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Rows ``2j`` = gate ``j``, ``2j+1`` = up ``j`` (the layout the GLU epilogue reads)."""
    return torch.stack([w_gate, w_up], dim=1).reshape(-1, *w_gate.shape[1:])


def gemm(x, w, *, bias=None, residual=None, res_mod=0, col_gate=None, row_scale=None,
         act="none", glu=False, a_scale=None, w_scale=None, out_dtype=torch.bfloat16,
         sumsq: Optional[torch.Tensor] = None):
    acc = x.float() @ w.float().t()
    if row_scale is not None:
        acc = acc * row_scale.float()[:, None]
    if a_scale is not None:
        acc = acc * a_scale.float()[:, None] * w_scale.float()[None, :]
    if bias is not None:
        acc = acc + bias.float()[None, :]
    if glu:
        acc = act_fn(acc[:, 0::2], act) * acc[:, 1::2]
    else:
        acc = act_fn(acc, act)
    if col_gate is not None:
        acc = acc * col_gate.float()[None, :]
    if residual is not None:
        r = residual.float()
        if res_mod:
            idx = torch.arange(acc.shape[0], device=acc.device) % res_mod
            r = r[idx]
        acc = acc + r
    out = acc.to(out_dtype)
    if sumsq is not None:
        sumsq += out.float().pow(2).sum(-1)
    return out


def attention(q, k, v, q_start, q_len, kv_indptr, kv_len, *, kv_indices=None, causal=False,
              sm_scale=None):
    """q (T,Hq,D); k/v pools (R,Hkv,D). Returns (T,Hq,D) in q.dtype; rows outside any sequence are 0."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    if sm_scale is None:
        sm_scale = D ** -0.5
    out = torch.zeros_like(q)
    for b in range(len(q_len)):
        qs, ql, ks, kl = int(q_start[b]), int(q_len[b]), int(kv_indptr[b]), int(kv_len[b])
        if ql == 0:
            continue
        if kv_indices is not None:
            rows = kv_indices[ks:ks + kl].long()
        else:
            rows = torch.arange(ks, ks + kl, device=q.device)
        qq = q[qs:qs + ql].float()                        # (ql, Hq, D)
        kk = k[rows].float().repeat_interleave(g, dim=1)  # (kl, Hq, D)
        vv = v[rows].float().repeat_interleave(g, dim=1)
        s = torch.einsum("qhd,khd->hqk", qq, kk) * sm_scale
        if causal:
            qi = torch.arange(ql, device=q.device)[:, None] + (kl - ql)
            kj = torch.arange(kl, device=q.device)[None, :]
            s = s.masked_fill(kj > qi, float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p)
        o = torch.einsum("hqk,khd->qhd", p, vv)
        out[qs:qs + ql] = o.to(q.dtype)
    return out


def rms_norm(x, weight=None, eps=1e-6, gemma=False):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.float()
        y = y * (1.0 + w if gemma else w)
    return y.to(x.dtype)


def layer_norm(x, weight, bias, eps=1e-6):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps).to(x.dtype)


def ada_rms_norm(x, mod, eps=1e-6):
    """x (..., D); mod broadcastable (..., 3D) = scale | shift | gate. Returns (y, gate)."""
    D = x.shape[-1]
    scale, shift, gate = mod.float().split(D, dim=-1)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = y * (1.0 + scale) + shift
    return y.to(x.dtype), gate.to(x.dtype)


def rope_cos_sin(positions: torch.Tensor, rot_dim: int, theta: float = 10000.0) -> torch.Tensor:
    """(P,) positions -> (P, rot_dim) fp32 table ``cos(rot_dim/2) | sin(rot_dim/2)``."""
    half = rot_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=positions.device) / half))
    ang = positions.float()[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1)


def apply_rope(x: torch.Tensor, cos_sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE. x (T, H, D); cos_sin (T, rot_dim)."""
    rot = cos_sin.shape[-1]
    half = rot // 2
    c = cos_sin[:, None, :half].float()
    s = cos_sin[:, None, half:].float()
    xf = x.float()
    x1, x2, rest = xf[..., :half], xf[..., half:rot], xf[..., rot:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1).to(x.dtype)


def embedding(ids, table, lo=0, hi=None, scale=1.0):
    if hi is None:
        hi = lo + table.shape[0]
    mask = (ids >= lo) & (ids < hi)
    idx = torch.where(mask, ids - lo, torch.zeros_like(ids))
    out = table[idx].float() * scale
    out = out * mask[..., None]
    return out.to(table.dtype)


def im2col(pix: torch.Tensor, p: int, kpad: int) -> torch.Tensor:
    n, c, h, w = pix.shape
    x = pix.reshape(n, c, h // p, p, w // p, p).permute(0, 2, 4, 1, 3, 5).reshape(n * (h // p) * (w // p), c * p * p)
    return F.pad(x, (0, kpad - c * p * p))


def gated_act(x, act, interleaved=False):
    xf = x.float()
    if interleaved:
        g, u = xf[..., 0::2], xf[..., 1::2]
    else:
        g, u = xf.chunk(2, dim=-1)
    return (act_fn(g, act) * u).to(x.dtype)


def cfg_combine(cond, uncond, g):
    return (uncond.float() + g * (cond.float() - uncond.float())).to(cond.dtype)


def quant_fp8(x: torch.Tensor, block: int = 0):
    xf = x.float()
    if block:
        r, d = xf.shape
        xb = xf.reshape(r, d // block, block)
        sc = xb.abs().amax(-1).clamp_min(1e-12) / 448.0
        y = (xb / sc[..., None]).reshape(r, d)
    else:
        sc = xf.abs().amax(-1).clamp_min(1e-12) / 448.0
        y = xf / sc[:, None]
    return y.clamp(-448, 448).to(torch.float8_e4m3fn), sc


def sinusoidal_time_embedding(t: torch.Tensor, dim: int, min_period: float, max_period: float) -> torch.Tensor:
    """Flow-matching time embedding ``sin | cos`` with log-spaced periods (fp32)."""
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float32, device=t.device)
    period = min_period * (max_period / min_period) ** frac
    ang = (2.0 * math.pi / period)[None, :] * t.float()[:, None]
    return torch.cat([ang.sin(), ang.cos()], dim=1)
