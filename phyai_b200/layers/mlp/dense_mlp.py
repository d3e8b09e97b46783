"""Dense MLP block, gated or plain, tensor-parallel.

* gated:  ``down(act(gate(x)) * up(x))`` with gate/up fused in one column-parallel weight whose
  rows interleave (gate_j, up_j), so the GEMM epilogue applies the gated activation and the
  intermediate ``(M, 2I)`` tensor never exists on the CUDA path;
* plain:  ``fc2(act(fc1(x)))`` with the activation fused into fc1's epilogue.
``moe_mlp`` has no counterpart here: the reference file is empty (phyai/src/phyai/layers/mlp/moe_mlp.py).
Reference: phyai/src/phyai/layers/mlp/dense_mlp.py:79-276.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops
from ...engine_config import get_engine_config
from ...ops import ref
from ..linear import ColumnParallelLinear, MergedColumnParallelLinear, RowParallelLinear

_GATED = {"silu": "silu", "swish": "silu", "gelu": "gelu", "gelu_tanh": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh"}


class DenseMLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, *, gated: bool = True, activation: str = "silu",
                 bias: bool = False, params_dtype: torch.dtype | None = None, axis: str = "tp", sp_axis: str | None = None,
                 prefix: str = "", hf_names: tuple[str, ...] | None = None, mesh=None) -> None:
        super().__init__()
        if activation not in _GATED:
            raise ValueError(f"unknown MLP activation {activation!r}")
        self.gated, self.activation = gated, _GATED[activation]
        kw = dict(bias=bias, params_dtype=params_dtype, axis=axis, mesh=mesh)
        if gated:
            g, u, d = hf_names or ("gate_proj", "up_proj", "down_proj")
            self.gate_up_proj = MergedColumnParallelLinear(hidden_size, [intermediate_size] * 2, hf_legs=(g, u),
                                                           interleave=True, sp_axis=sp_axis,
                                                           prefix=f"{prefix}.gate_up_proj" if prefix else "gate_up_proj", **kw)
            self.down_proj = RowParallelLinear(intermediate_size, hidden_size, sp_axis=sp_axis,
                                               prefix=f"{prefix}.{d}" if prefix else d, **kw)
        else:
            a, b = hf_names or ("fc1", "fc2")
            self.fc1 = ColumnParallelLinear(hidden_size, intermediate_size, sp_axis=sp_axis,
                                            prefix=f"{prefix}.{a}" if prefix else a, **kw)
            self.fc2 = RowParallelLinear(intermediate_size, hidden_size, sp_axis=sp_axis,
                                         prefix=f"{prefix}.{b}" if prefix else b, **kw)

    def _fusable(self, x: torch.Tensor, lin) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and lin.spec.spec_id == "bf16" and lin.sp_axis is None
                and get_engine_config().resolved_backend("linear") == "b200" and x.shape[-1] % 8 == 0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if self.gated:
            gu = self.gate_up_proj
            if self._fusable(x2, gu):
                h = ops.gemm(x2.contiguous(), gu.weight, bias=gu.bias, act=self.activation, glu=True)
            else:
                y, _ = gu(x2)
                h = ref.gated_act(y, self.activation, interleaved=True)
            out, _ = self.down_proj(h)
        else:
            if self._fusable(x2, self.fc1):
                h = ops.gemm(x2.contiguous(), self.fc1.weight, bias=self.fc1.bias, act=self.activation)
            else:
                y, _ = self.fc1(x2)
                h = ref.act_fn(y.float(), self.activation).to(y.dtype)
            out, _ = self.fc2(h)
        return out.reshape(*lead, -1)


__all__ = ["DenseMLP"]
