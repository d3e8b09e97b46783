"""Normalisation layers: RMSNorm, GemmaRMSNorm ((1+w)), LayerNorm, AdaRMSNorm.

On CUDA bf16 rows the ``b200`` backend runs the single-pass kernels of
``csrc/ops.cu``; everything else (CPU, fp32 parity paths) runs the plain PyTorch
restatement. ``forward(x, residual)`` fuses ``residual += x`` with the norm and
returns ``(y, residual)``. Reference: phyai/src/phyai/layers/layer_norm.py:64-603.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..engine_config import get_engine_config, resolve_engine_defaults
from ..ops import ref
from .linear import ReplicatedLinear


def _use_kernel(backend: str, x: torch.Tensor) -> bool:
    return backend == "b200" and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


class RMSNorm(nn.Module):
    gemma = False

    def __init__(self, hidden_size: int, eps: float = 1e-6, *, backend: str | None = None,
                 dtype: torch.dtype | None = None, device=None, prefix: str = "") -> None:
        super().__init__()
        dtype, _, backend = resolve_engine_defaults(dtype, None, backend)
        device = device if device is not None else get_engine_config().device.target
        self.hidden_size, self.variance_epsilon, self.backend, self.prefix = hidden_size, eps, backend, prefix
        init = torch.zeros if self.gemma else torch.ones
        self.weight = nn.Parameter(init(hidden_size, dtype=dtype, device=device), requires_grad=False)
        if prefix:
            self.weight.hf_keys = {f"{prefix}.weight": None}

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        if _use_kernel(self.backend, x):
            x2 = x.reshape(-1, x.shape[-1])
            mode = "gemma_rms" if self.gemma else "rms"
            if residual is None:
                return ops.norm(x2, mode, weight=self.weight, eps=self.variance_epsilon).reshape(x.shape)
            r2 = residual.reshape(-1, x.shape[-1])
            y = ops.norm(x2, mode, weight=self.weight, residual=r2, eps=self.variance_epsilon)
            return y.reshape(x.shape), residual
        if residual is not None:
            residual.add_(x)
            return ref.rms_norm(residual, self.weight, self.variance_epsilon, self.gemma), residual
        return ref.rms_norm(x, self.weight, self.variance_epsilon, self.gemma)


class GemmaRMSNorm(RMSNorm):
    gemma = True


class LayerNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, *, bias: bool = True, backend: str | None = None,
                 dtype: torch.dtype | None = None, device=None, prefix: str = "") -> None:
        """``bias=False``: the shift stays zero and expects no checkpoint tensor."""
        super().__init__()
        dtype, _, backend = resolve_engine_defaults(dtype, None, backend)
        device = device if device is not None else get_engine_config().device.target
        self.hidden_size, self.eps, self.backend, self.prefix = hidden_size, eps, backend, prefix
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=device), requires_grad=False)
        self.has_bias = bool(bias)
        if prefix:
            self.weight.hf_keys = {f"{prefix}.weight": None}
            if bias:
                self.bias.hf_keys = {f"{prefix}.bias": None}
        if not bias:
            self.bias.optional = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if _use_kernel(self.backend, x):
            return ops.norm(x.reshape(-1, x.shape[-1]), "layer", weight=self.weight, bias=self.bias,
                            eps=self.eps).reshape(x.shape)
        return ref.layer_norm(x, self.weight, self.bias, self.eps)


class AdaRMSNorm(nn.Module):
    """``x_hat * (1 + scale) + shift`` with ``(scale, shift, gate) = dense(cond).chunk(3)``.

    ``forward(x, cond)`` projects the condition; ``forward(x, modulation=row)`` applies a
    row precomputed with :meth:`project_modulation` (kept out of captured graphs).
    Returns ``(y, gate)``; ``gate`` broadcasts against ``y``.
    """

    def __init__(self, hidden_size: int, cond_dim: int, eps: float = 1e-6, backend: str | None = None, *,
                 dtype: torch.dtype | None = None, device=None, prefix: str = "") -> None:
        super().__init__()
        if hidden_size <= 0 or cond_dim <= 0:
            raise ValueError("AdaRMSNorm: hidden_size and cond_dim must be positive")
        dtype, _, backend = resolve_engine_defaults(dtype, None, backend)
        self.hidden_size, self.cond_dim, self.variance_epsilon = hidden_size, cond_dim, eps
        self.backend, self.prefix = backend, prefix
        self.dense = ReplicatedLinear(cond_dim, 3 * hidden_size, bias=True, params_dtype=dtype, device=device,
                                      prefix=f"{prefix}.dense" if prefix else "")
        nn.init.zeros_(self.dense.weight)
        nn.init.zeros_(self.dense.bias)

    def project_modulation(self, conds: torch.Tensor) -> torch.Tensor:
        if conds.shape[-1] != self.cond_dim:
            raise ValueError(f"AdaRMSNorm: conds last dim {conds.shape[-1]} != cond_dim {self.cond_dim}")
        with torch.no_grad():
            return self.dense(conds)[0].contiguous()

    def forward(self, x: torch.Tensor, cond: torch.Tensor | None = None, *, modulation: torch.Tensor | None = None):
        if x.shape[-1] != self.hidden_size:
            raise ValueError(f"AdaRMSNorm: x last dim {x.shape[-1]} != hidden_size {self.hidden_size}")
        if (cond is None) == (modulation is None):
            raise ValueError("AdaRMSNorm: pass exactly one of cond / modulation")
        mod = modulation if modulation is not None else self.dense(cond)[0]
        if mod.dim() == x.dim() - 1:      # (B, 3D) against (B, S, D)
            mod = mod.unsqueeze(-2)
        D = self.hidden_size
        rows = x.numel() // D
        mrows = mod.numel() // (3 * D)
        if _use_kernel(self.backend, x) and mod.dtype == torch.bfloat16 and rows % mrows == 0 and mod.is_contiguous():
            y = ops.norm(x.reshape(rows, D), "ada_rms", mod=mod.reshape(mrows, 3 * D), group=rows // mrows,
                         eps=self.variance_epsilon).reshape(x.shape)
            return y, mod[..., 2 * D:]
        return ref.ada_rms_norm(x, mod, self.variance_epsilon)


__all__ = ["RMSNorm", "GemmaRMSNorm", "LayerNorm", "AdaRMSNorm"]
