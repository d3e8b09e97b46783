"""NVFP4 linear on the block-scaled tensor cores: e2m1 operands, one ue4m3 scale per 16 elements of K, fp32 global
scales. Kernels: ``csrc/cutlass/`` (built into ``phyai_b200/_blockscaled``; optional: without it NVFP4 layers
run through the dequantising reference path).

Reference: FlashInfer ``mm_fp4`` + ``nvfp4_quantize`` (phyai/src/phyai/layers/linear/backends/flashinfer.py:163-200).
"""

from __future__ import annotations

from typing import Optional

import torch

_EXT = None
_TRIED = False
_WORKSPACE: dict[torch.device, torch.Tensor] = {}
_ACT_BUFFERS: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def ext():
    """The native module, or ``None`` where it was not built."""
    global _EXT, _TRIED
    if not _TRIED:
        _TRIED = True
        try:
            from .. import _blockscaled as m  # type: ignore[attr-defined]

            _EXT = m
        except ImportError:
            _EXT = None
    return _EXT


def available() -> bool:
    return ext() is not None and torch.cuda.is_available()


def _workspace(dev: torch.device) -> torch.Tensor:
    ws = _WORKSPACE.get(dev)
    if ws is None:
        ws = _WORKSPACE[dev] = torch.zeros(32 << 20, dtype=torch.uint8, device=dev)
    return ws


def quantize_activation(x: torch.Tensor, global_scale: float = 1.0, *, cached: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``(M, K)`` -> packed e2m1 ``(M, K/2)`` and its ue4m3 block scales in the interleaved 128 x 4 layout the MMA
    reads (``x ~ e2m1 * scale * global_scale``). ``cached``: reuse one pair of buffers per shape (a serving loop)."""
    M, K = x.shape
    key = (x.device, M, K)
    bufs = _ACT_BUFFERS.get(key) if cached else None
    if bufs is None:
        q = torch.empty(M, K // 2, dtype=torch.uint8, device=x.device)
        sf = torch.zeros(ext().scale_bytes(M, K), dtype=torch.uint8, device=x.device)      # padding stays zero
        bufs = (q, sf)
        if cached:
            _ACT_BUFFERS[key] = bufs
    ext().quantize_act(x, float(global_scale), bufs[0], bufs[1])
    return bufs


def swizzle_scales(scales: torch.Tensor, K: int) -> torch.Tensor:
    """Row-major one-byte block scales ``(rows, K/16)`` -> the interleaved layout (a flat uint8 buffer)."""
    return ext().swizzle_scales(scales.contiguous().view(torch.uint8), K)


def gemm_nvfp4(x4: torch.Tensor, sfx: torch.Tensor, w4: torch.Tensor, sfw: torch.Tensor, alpha: float, *,
               out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, tile: int = 0) -> torch.Tensor:
    """``alpha * (x4 . sfx) @ (w4 . sfw)^T`` in bf16; scales already in the interleaved layout."""
    if out is None:
        out = torch.empty(x4.shape[0], w4.shape[0], dtype=torch.bfloat16, device=x4.device)
    ext().gemm(x4, sfx, w4, sfw, out, float(alpha), bias, _workspace(x4.device), tile)
    return out


def linear(x: torch.Tensor, layer, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """An ``Nvfp4Spec`` layer applied to bf16 rows: the weight scales are re-laid once per layer, the activation is
    quantised with the layer's ``input_scale`` as its global scale."""
    prep = getattr(layer, "_nvfp4_prepared", None)
    K = layer.weight.shape[1] * 2
    if prep is None or prep[0].device != layer.weight.device:
        prep = (swizzle_scales(layer.weight_scale.data, K), float(layer.weight_global_scale.item()), float(layer.input_scale.item()))
        layer._nvfp4_prepared = prep
    sfw, gw, gx = prep
    q, sfx = quantize_activation(x, gx)
    b = None if bias is None else bias.to(torch.bfloat16)
    return gemm_nvfp4(q, sfx, layer.weight.data, sfw, gx * gw, bias=b)


def ref_gemm_nvfp4(x4, sfx_linear, w4, sfw_linear, alpha: float) -> torch.Tensor:
    """fp32 restatement from row-major scales: dequantise both operands, ordinary product."""
    from ..layers.quant.specs import Nvfp4Spec

    one = torch.ones(1, device=x4.device)
    xf = Nvfp4Spec.dequantize(x4, sfx_linear, one)
    wf = Nvfp4Spec.dequantize(w4, sfw_linear, one)
    return alpha * (xf @ wf.t())


def unswizzle_scales(sf: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """Inverse of :func:`swizzle_scales` in PyTorch (tests): flat interleaved buffer -> ``(rows, K/16)`` e4m3."""
    nkb = K // 16
    kbp = (K + 63) // 64 * 4
    r = torch.arange(rows, device=sf.device)[:, None]
    kb = torch.arange(nkb, device=sf.device)[None, :]
    off = ((r // 128) * (kbp // 4) + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    return sf[off.reshape(-1)].reshape(rows, nkb).view(torch.float8_e4m3fn)


__all__ = ["available", "quantize_activation", "swizzle_scales", "unswizzle_scales", "gemm_nvfp4", "linear", "ref_gemm_nvfp4"]
