"""Convolution wrappers with checkpoint loaders.

``Conv1d / Conv2d / Conv3d / ConvTranspose1d`` own their parameters with checkpoint keys,
support asymmetric (causal) padding given per side, and can fold a weight-normed
checkpoint (``weight_g``, ``weight_v``) into a plain weight at load time.
Reference: phyai/src/phyai/layers/conv.py:59-432.
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..engine_config import get_engine_config
from ..weights import shards


def _tuple(v, n: int) -> tuple[int, ...]:
    return tuple(v) if isinstance(v, (tuple, list)) else (int(v),) * n


class _ConvNd(nn.Module):
    nd = 2
    transposed = False

    def __init__(self, in_channels: int, out_channels: int, kernel_size, *, stride=1, padding=0, dilation=1,
                 groups: int = 1, bias: bool = True, pad_sides: Sequence[int] | None = None, pad_mode: str = "constant",
                 weight_norm: bool = False, dtype: torch.dtype | None = None, device=None, prefix: str = "") -> None:
        super().__init__()
        cfg = get_engine_config()
        dtype = dtype or cfg.device.params_dtype
        device = device if device is not None else cfg.device.target
        n = self.nd
        self.kernel_size, self.stride = _tuple(kernel_size, n), _tuple(stride, n)
        self.padding, self.dilation, self.groups = _tuple(padding, n), _tuple(dilation, n), groups
        # explicit per-side padding (last dim first, as F.pad wants it); used for causal convs
        self.pad_sides, self.pad_mode = (tuple(pad_sides) if pad_sides is not None else None), pad_mode
        shape = ((in_channels, out_channels // groups) if self.transposed else (out_channels, in_channels // groups))
        self.weight = nn.Parameter(torch.empty(*shape, *self.kernel_size, dtype=dtype, device=device), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(out_channels, dtype=dtype, device=device), requires_grad=False) if bias else None
        if prefix:
            if weight_norm:
                keys = {f"{prefix}.weight_g": "g", f"{prefix}.weight_v": "v",
                        f"{prefix}.parametrizations.weight.original0": "g", f"{prefix}.parametrizations.weight.original1": "v"}
                self.weight.hf_keys = keys
                self.weight.weight_loader = shards.weight_norm_fold(0)
                self.weight.hf_alternatives = True
            else:
                self.weight.hf_keys = {f"{prefix}.weight": None}
            if self.bias is not None:
                self.bias.hf_keys = {f"{prefix}.bias": None}

    def _pad(self, x: torch.Tensor) -> torch.Tensor:
        if self.pad_sides is None:
            return x
        return F.pad(x, self.pad_sides, mode=self.pad_mode)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[self.nd]
        pad = (0,) * self.nd if self.pad_sides is not None else self.padding
        w = self.weight.to(x.dtype)
        b = None if self.bias is None else self.bias.to(x.dtype)
        return fn(self._pad(x), w, b, self.stride, pad, self.dilation, self.groups)


class Conv1d(_ConvNd):
    nd = 1


class Conv2d(_ConvNd):
    nd = 2


class Conv3d(_ConvNd):
    nd = 3


class ConvTranspose1d(_ConvNd):
    nd = 1
    transposed = True

    def __init__(self, *a, output_padding: int = 0, **kw) -> None:
        super().__init__(*a, **kw)
        self.output_padding = output_padding

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b = None if self.bias is None else self.bias.to(x.dtype)
        return F.conv_transpose1d(x, self.weight.to(x.dtype), b, self.stride, self.padding, self.output_padding,
                                  self.groups, self.dilation)


class PositionEmbedding(nn.Module):
    """Learned position table added to a token grid (SigLIP)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, dtype=None, device=None, prefix: str = "") -> None:
        super().__init__()
        cfg = get_engine_config()
        self.weight = nn.Parameter(torch.zeros(num_embeddings, embedding_dim, dtype=dtype or cfg.device.params_dtype,
                                               device=device if device is not None else cfg.device.target),
                                   requires_grad=False)
        if prefix:
            self.weight.hf_keys = {f"{prefix}.weight": None}

    def forward(self) -> torch.Tensor:
        return self.weight


__all__ = ["Conv1d", "Conv2d", "Conv3d", "ConvTranspose1d", "PositionEmbedding"]
