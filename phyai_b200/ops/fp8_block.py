"""Block-scaled fp8 linear: e4m3 activations with one fp32 scale per 1x128 block, e4m3 weights with one per
128x128 block (the layout block-quantised checkpoints ship). Kernel: ``csrc/gemm_fp8_block.cu``."""

from __future__ import annotations

from typing import Optional

import torch

from . import ACT, ext


def gemm_fp8_block(x8: torch.Tensor, x_scale: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor, out: Optional[torch.Tensor] = None, *,
                   bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None, col_gate: Optional[torch.Tensor] = None,
                   act: str | None = "none", glu: bool = False, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``x8`` (M, K) e4m3 with ``x_scale`` (M, K/128); ``w8`` (N, K) e4m3 with ``w_scale`` (ceil(N/128), K/128)."""
    M, N = x8.shape[0], w8.shape[0]
    if out is None:
        out = torch.empty((M, N // 2 if glu else N), dtype=out_dtype, device=x8.device)
    ext().gemm_fp8_block(x8, w8, out, x_scale.contiguous(), w_scale.contiguous(), bias, residual, col_gate, ACT[act], glu)
    return out


def ref_gemm_fp8_block(x8, x_scale, w8, w_scale, bias=None) -> torch.Tensor:
    """fp32 restatement: dequantise both operands block by block, then an ordinary product."""
    M, K = x8.shape
    N = w8.shape[0]
    xf = x8.float().reshape(M, K // 128, 128) * x_scale.float()[..., None]
    ws = w_scale.float().repeat_interleave(128, dim=0)[:N]                      # (N, K/128)
    wf = w8.float().reshape(N, K // 128, 128) * ws[..., None]
    y = xf.reshape(M, K) @ wf.reshape(N, K).t()
    return y if bias is None else y + bias.float()


def quantize_weight_block(w: torch.Tensor, block: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """(N, K) float -> e4m3 weight and (ceil(N/128), K/128) scales (amax / 448 per block)."""
    N, K = w.shape
    nb = -(-N // block)
    wp = torch.zeros(nb * block, K, dtype=torch.float32, device=w.device)
    wp[:N] = w.float()
    blocks = wp.reshape(nb, block, K // block, block)
    scale = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12) / 448.0
    q = (blocks / scale[:, None, :, None]).clamp(-448, 448).reshape(nb * block, K)[:N].to(torch.float8_e4m3fn)
    return q, scale


def quantize_rows_into(x: torch.Tensor, y8: torch.Tensor, scale: torch.Tensor, block: int = 128) -> None:
    """bf16 rows -> e4m3 with one scale per 1 x ``block`` group, into caller-owned buffers (no allocation:
    what a captured serving plan calls between a bf16 producer and a block-scaled GEMM)."""
    ext().quant_fp8(x, y8, scale, block)


def layer_weight_fp8(layer) -> tuple[torch.Tensor, torch.Tensor]:
    """Block-scaled e4m3 weight and scales of a linear layer: taken as stored when the layer was built from a
    block-fp8 checkpoint, quantised here (128 x 128 blocks, amax / 448) when it holds bf16 / fp16 / fp32."""
    w = layer.weight
    if w.dtype == torch.float8_e4m3fn:
        ws = getattr(layer, "weight_scale", None)
        if ws is None or ws.dim() != 2:
            raise ValueError("fp8 layer without 2-D block scales: only fp8_block_128_128 weights can be served as stored")
        return w.data, ws.data.float().contiguous()
    if w.shape[1] % 128:
        raise ValueError(f"block-scaled fp8 needs in_features % 128 == 0, got {w.shape[1]}")
    return quantize_weight_block(w.data)


__all__ = ["gemm_fp8_block", "ref_gemm_fp8_block", "quantize_weight_block", "quantize_rows_into", "layer_weight_fp8"]
