"""Weight specs: how a linear layer allocates, post-processes and applies a scheme.

A spec owns the parameters it registers on the layer (``weight`` plus scale
tensors), the post-load fixups, the activation quantiser and a plain-PyTorch
reference ``apply`` (dequantise + matmul) that every kernel is tested against.

Reference: phyai/src/phyai/layers/quant/{base,bf16,fp8,nvfp4,linear,materialize}.py.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import NamedTuple, Protocol, runtime_checkable

import torch
import torch.nn as nn
import torch.nn.functional as F

from .scheme import Granularity, QDType, QuantScheme

FP8_MAX = 448.0
FP4_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


class ActivationView(NamedTuple):
    """What a kernel gets from a spec that quantises activations in front of the product."""

    x: torch.Tensor
    x_scale: torch.Tensor | None
    granularity: Granularity


@runtime_checkable
class WeightSpec(Protocol):
    """How one weight format lives in a linear layer: which parameters it allocates, what it fixes up after loading and
    the PyTorch statement of the product (the oracle of the kernel tests). Reference:
    phyai/src/phyai/layers/quant/base.py."""

    spec_id: str
    min_sm: int

    def allocate(self, layer: nn.Module, req: "AllocationRequest") -> None: ...

    def process_after_loading(self, layer: nn.Module) -> None: ...

    def reference_apply(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor: ...


@runtime_checkable
class LinearActivationQuant(Protocol):
    """Specs whose kernels take quantised activations (``isinstance(spec, LinearActivationQuant)`` instead of looking at
    spec ids). Reference: phyai/src/phyai/layers/quant/linear.py:34-48; here ``quantize_activation(x)`` returns the
    ``(values, scales)`` pair the CUDA quantiser produces and ``activation_view`` wraps it with its granularity."""

    needs_act_quant: bool

    def quantize_activation(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]: ...

    def activation_view(self, x: torch.Tensor, layer: nn.Module | None = None) -> ActivationView: ...


@dataclass(frozen=True)
class AllocationRequest:
    out_features: int
    in_features: int
    params_dtype: torch.dtype
    device: torch.device | str


class Bf16Spec:
    """Unquantised weights in the engine dtype (bf16 / fp16 / fp32)."""

    spec_id = "bf16"
    min_sm = 0

    def allocate(self, layer: nn.Module, req: AllocationRequest) -> None:
        layer.weight = nn.Parameter(torch.empty(req.out_features, req.in_features, dtype=req.params_dtype,
                                                device=req.device), requires_grad=False)

    def process_after_loading(self, layer: nn.Module) -> None:
        pass

    def reference_apply(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        return F.linear(x, layer.weight.to(x.dtype), None if bias is None else bias.to(x.dtype))


class Fp8Spec:
    """e4m3 weights with per-tensor, per-channel or 2-D block scales; activations are
    quantised on the fly (per token, or per 1 x block_k group for block scales)."""

    min_sm = 89
    needs_act_quant = True

    def __init__(self, scheme: QuantScheme) -> None:
        self.scheme = scheme
        self.granularity = scheme.weight.granularity
        self.block = scheme.weight.block_shape
        self.spec_id = scheme.spec_id

    def allocate(self, layer: nn.Module, req: AllocationRequest) -> None:
        n, k = req.out_features, req.in_features
        layer.weight = nn.Parameter(torch.zeros(n, k, dtype=torch.float8_e4m3fn, device=req.device), requires_grad=False)
        if self.granularity is Granularity.BLOCK:
            bn, bk = self.block  # type: ignore[misc]
            shape = ((n + bn - 1) // bn, (k + bk - 1) // bk)
        elif self.granularity is Granularity.PER_CHANNEL:
            shape = (n,)
        else:
            shape = (1,)  # per-tensor in the checkpoint; fanned out to per-channel after load
        layer.weight_scale = nn.Parameter(torch.ones(shape, dtype=torch.float32, device=req.device), requires_grad=False)
        layer.input_scale = nn.Parameter(torch.ones(1, dtype=torch.float32, device=req.device), requires_grad=False)

    def process_after_loading(self, layer: nn.Module) -> None:
        ws = layer.weight_scale
        if self.granularity is Granularity.PER_TENSOR and ws.numel() != layer.weight.shape[0]:
            # one scale per fused leg (or one overall) -> one scale per output channel
            n = layer.weight.shape[0]
            legs = ws.numel()
            layer.weight_scale = nn.Parameter(ws.data.reshape(legs, 1).expand(legs, n // legs).reshape(n).contiguous(),
                                              requires_grad=False)

    def quantize_weight(self, w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        wf = w.float()
        if self.granularity is Granularity.BLOCK:
            bn, bk = self.block  # type: ignore[misc]
            n, k = wf.shape
            pn, pk = (-n) % bn, (-k) % bk
            wp = F.pad(wf, (0, pk, 0, pn)).reshape((n + pn) // bn, bn, (k + pk) // bk, bk)
            sc = wp.abs().amax(dim=(1, 3)).clamp_min(1e-12) / FP8_MAX
            q = (wp / sc[:, None, :, None]).reshape(n + pn, k + pk)[:n, :k]
            return q.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), sc
        if self.granularity is Granularity.PER_CHANNEL:
            sc = wf.abs().amax(dim=1).clamp_min(1e-12) / FP8_MAX
            return (wf / sc[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), sc
        sc = (wf.abs().amax().clamp_min(1e-12) / FP8_MAX).reshape(1)
        return (wf / sc).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), sc

    def quantize_activation(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Dynamic: per token, or per (token, block_k group) for block-scaled weights."""
        xf = x.float()
        if self.granularity is Granularity.BLOCK:
            bk = self.block[1]  # type: ignore[index]
            m, k = xf.shape
            pk = (-k) % bk
            xp = F.pad(xf, (0, pk)).reshape(m, (k + pk) // bk, bk)
            sc = xp.abs().amax(-1).clamp_min(1e-12) / FP8_MAX
            q = (xp / sc[..., None]).reshape(m, k + pk)[:, :k]
            return q.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), sc
        sc = xf.abs().amax(-1).clamp_min(1e-12) / FP8_MAX
        return (xf / sc[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), sc

    def activation_view(self, x: torch.Tensor, layer: nn.Module | None = None) -> ActivationView:
        q, sc = self.quantize_activation(x.reshape(-1, x.shape[-1]))
        return ActivationView(q, sc, Granularity.GROUP if self.granularity is Granularity.BLOCK else Granularity.PER_TOKEN)

    def dequant_weight(self, layer: nn.Module) -> torch.Tensor:
        w = layer.weight.float()
        s = layer.weight_scale.float()
        if self.granularity is Granularity.BLOCK:
            bn, bk = self.block  # type: ignore[misc]
            s = s.repeat_interleave(bn, 0)[: w.shape[0]].repeat_interleave(bk, 1)[:, : w.shape[1]]
            return w * s
        if s.numel() == 1:
            return w * s
        return w * s[:, None]

    def reference_apply(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        q, sc = self.quantize_activation(x2)
        if self.granularity is Granularity.BLOCK:
            bk = self.block[1]  # type: ignore[index]
            xd = q.float() * sc.repeat_interleave(bk, 1)[:, : x2.shape[1]]
        else:
            xd = q.float() * sc[:, None]
        y = xd @ self.dequant_weight(layer).t()
        if bias is not None:
            y = y + bias.float()
        return y.to(x.dtype).reshape(*lead, -1)


class Nvfp4Spec:
    """NVFP4: e2m1 values packed two per byte, one e4m3 scale per 16 elements, one fp32
    global scale. Weights are quantised at load when the checkpoint is not packed."""

    min_sm = 100
    spec_id = "nvfp4_block_16"
    group = 16

    def __init__(self, scheme: QuantScheme | None = None, layout: str = "linear") -> None:
        if layout not in ("linear", "128x4"):
            raise ValueError(f"unknown NVFP4 scale layout {layout!r}")
        self.scheme = scheme
        self.layout = layout

    def allocate(self, layer: nn.Module, req: AllocationRequest) -> None:
        n, k = req.out_features, req.in_features
        if k % self.group:
            raise ValueError(f"NVFP4 needs in_features divisible by {self.group}, got {k}")
        layer.weight = nn.Parameter(torch.zeros(n, k // 2, dtype=torch.uint8, device=req.device), requires_grad=False)
        layer.weight_scale = nn.Parameter(torch.zeros(n, k // self.group, dtype=torch.float8_e4m3fn, device=req.device),
                                          requires_grad=False)
        layer.weight_global_scale = nn.Parameter(torch.ones(1, dtype=torch.float32, device=req.device), requires_grad=False)
        layer.input_scale = nn.Parameter(torch.ones(1, dtype=torch.float32, device=req.device), requires_grad=False)

    def process_after_loading(self, layer: nn.Module) -> None:
        pass

    @staticmethod
    def quantize(w: torch.Tensor, group: int = 16) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """-> (packed uint8 (n, k/2), e4m3 block scales (n, k/group), fp32 global scale)."""
        wf = w.float()
        n, k = wf.shape
        gs = (wf.abs().amax().clamp_min(1e-12) / (6.0 * FP8_MAX)).reshape(1)
        blk = wf.reshape(n, k // group, group)
        bs = (blk.abs().amax(-1) / 6.0 / gs).clamp(max=FP8_MAX).to(torch.float8_e4m3fn)
        denom = (bs.float() * gs).clamp_min(1e-12)[..., None]
        v = (blk / denom).reshape(n, k)
        grid = FP4_VALUES.to(v.device)
        idx = (v.abs()[..., None] - grid).abs().argmin(-1).to(torch.uint8)
        code = idx | ((v < 0).to(torch.uint8) << 3)
        packed = code[:, 0::2] | (code[:, 1::2] << 4)
        return packed, bs, gs

    @staticmethod
    def dequantize(packed: torch.Tensor, bs: torch.Tensor, gs: torch.Tensor, group: int = 16) -> torch.Tensor:
        lo, hi = packed & 0xF, packed >> 4
        code = torch.stack([lo, hi], dim=-1).reshape(packed.shape[0], -1).long()
        grid = FP4_VALUES.to(packed.device)
        val = grid[code & 7] * torch.where((code & 8) > 0, -1.0, 1.0)
        return val * (bs.float() * gs.float()).repeat_interleave(group, 1)

    def load_full_precision(self, layer: nn.Module, w: torch.Tensor) -> None:
        p, bs, gs = self.quantize(w.to(layer.weight.device), self.group)
        layer.weight.data.copy_(p)
        layer.weight_scale.data.copy_(bs)
        layer.weight_global_scale.data.copy_(gs)

    def reference_apply(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        w = self.dequantize(layer.weight, layer.weight_scale, layer.weight_global_scale, self.group)
        y = x.float() @ w.t()
        if bias is not None:
            y = y + bias.float()
        return y.to(x.dtype)


def materialize(scheme: QuantScheme | None, sm: int | None = None):
    """Scheme -> spec object. SM support is checked lazily at kernel dispatch, not here."""
    if scheme is None or scheme.weight.dtype in (QDType.BF16, QDType.FP16):
        return Bf16Spec()
    if scheme.weight.dtype is QDType.NVFP4:
        return Nvfp4Spec(scheme)
    if scheme.weight.dtype in (QDType.FP8_E4M3, QDType.FP8_E5M2):
        return Fp8Spec(scheme)
    raise ValueError(f"no weight spec for {scheme}")


__all__ = ["ActivationView", "WeightSpec", "LinearActivationQuant", "AllocationRequest", "Bf16Spec", "Fp8Spec", "Nvfp4Spec", "materialize",
           "FP8_MAX"]
