"""Snake activation ``x + sin^2(alpha x) / beta`` with per-channel log-scale parameters.

The checkpoint stores ``log alpha`` / ``log beta``; ``post_load`` exponentiates them once. On CUDA
(bf16 / fp32, ``(B, C, T)``) the forward is one launch of ``snake_kernel`` (``csrc/ops.cu``); elsewhere the
PyTorch statement below. Reference: phyai/src/phyai/layers/activation.py:12-67.
"""

from __future__ import annotations

import torch
import torch.nn as nn


class Snake1d(nn.Module):
    def __init__(self, channels: int, *, logscale: bool = True, dtype: torch.dtype | None = None, device=None,
                 prefix: str = "") -> None:
        super().__init__()
        self.logscale = logscale
        self.alpha = nn.Parameter(torch.zeros(1, channels, 1, dtype=dtype, device=device), requires_grad=False)
        self.beta = nn.Parameter(torch.zeros(1, channels, 1, dtype=dtype, device=device), requires_grad=False)
        if prefix:
            self.alpha.hf_keys = {f"{prefix}.alpha": None}
            self.beta.hf_keys = {f"{prefix}.beta": None}
            for p in (self.alpha, self.beta):
                p.weight_loader = lambda param, t, sid=None: param.data.copy_(t.reshape(param.shape).to(param.dtype))
        self._ready = not logscale

    def post_load(self) -> None:
        if self.logscale and not self._ready:
            self.alpha.data = self.alpha.data.float().exp().to(self.alpha.dtype)
            self.beta.data = self.beta.data.float().exp().to(self.beta.dtype)
            self._ready = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a, b = self.alpha.float(), self.beta.float()
        if self.logscale and not self._ready:
            a, b = a.exp(), b.exp()
        if x.is_cuda and x.dim() == 3 and x.dtype in (torch.bfloat16, torch.float32):
            from .. import ops

            if ops.available():
                return ops.snake(x, a, b)
        xf = x.float()
        return (xf + torch.sin(a * xf).pow(2) / (b + 1e-9)).to(x.dtype)


__all__ = ["Snake1d"]
