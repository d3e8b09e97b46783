"""Replicated and tensor-parallel linear layers.

Every ``forward`` returns ``(y, bias_or_None)``: the second element is the bias the
caller must still add when the layer was built with ``skip_bias_add=True``.
Sharding (reference: phyai/src/phyai/layers/linear/layers.py:43-631):

* ``ColumnParallelLinear``        output dim split over ``axis``; optional sequence-parallel
                                  all-gather of the input and all-gather of the output
* ``MergedColumnParallelLinear``  several column-parallel projections in one weight (gate/up)
* ``QKVParallelLinear``           fused q/k/v; KV heads are replicated when tp > kv_heads
* ``RowParallelLinear``           input dim split; partial sums all-reduced (or reduce-scattered
                                  for sequence parallelism); bias added on rank 0 only

Weights keep the ``nn.Linear`` layout ``(out, in)``. Checkpoint keys and loaders hang
on the parameters for ``load_pretrained``.
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.nn as nn

from ... import parallel as P
from ...engine_config import get_engine_config
from ...parallel import state as pstate
from ...utils.cuda import sm_arch
from ...weights import shards
from ..quant.scheme import get_active_plan
from ..quant.specs import AllocationRequest, Bf16Spec, Nvfp4Spec, materialize
from .kernels import get_linear_dispatcher


def _axis_info(axis: str | None, mesh) -> tuple[int, int]:
    m = mesh if mesh is not None else pstate.default_mesh()
    if axis is None or m is None:
        return 0, 1
    return m.axis_local_rank(axis), m.axis_size(axis)


class LinearBase(nn.Module):
    def __init__(self, in_features: int, out_features: int, *, bias: bool = True, skip_bias_add: bool = False,
                 params_dtype: torch.dtype | None = None, spec: object | None = None, scheme: object | None = None,
                 device: torch.device | str | None = None, prefix: str = "") -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        cfg = get_engine_config()
        self.params_dtype = params_dtype or cfg.device.params_dtype
        self.skip_bias_add = skip_bias_add
        self.prefix = prefix
        self.device = device if device is not None else cfg.device.target
        # spec resolution: explicit spec > explicit scheme > active quant plan > unquantised
        if spec is not None:
            self.spec = spec
        elif scheme is not None:
            self.spec = materialize(scheme, sm_arch())
        else:
            plan = get_active_plan()
            resolved = plan.resolve(prefix, type(self)) if (plan is not None and prefix) else None
            self.spec = materialize(resolved, sm_arch()) if resolved is not None else Bf16Spec()
        self._bias_requested = bias

    # ------------------------------------------------------------- helpers
    def _allocate(self, n_local: int, k_local: int) -> None:
        self.spec.allocate(self, AllocationRequest(n_local, k_local, self.params_dtype, self.device))
        if self._bias_requested:
            self.bias = nn.Parameter(torch.zeros(n_local, dtype=self.params_dtype, device=self.device),
                                     requires_grad=False)
        else:
            self.register_parameter("bias", None)

    def _wire_weight(self, keys: dict[str, object], loader, full_shapes: dict[str, tuple[int, ...]] | None = None) -> None:
        w = self.weight
        w.hf_keys = keys
        if full_shapes:
            w.hf_shapes = full_shapes
        if isinstance(self.spec, Nvfp4Spec):
            # full-precision checkpoints are quantised as they arrive
            def nv_loader(param, tensor, shard_id, _l=loader, _self=self):
                if tensor.dtype == torch.uint8:
                    _l(param, tensor, shard_id)
                else:
                    tmp = nn.Parameter(torch.empty(param.shape[0], param.shape[1] * 2, dtype=torch.float32))
                    _l(tmp, tensor.float(), shard_id)
                    _self.spec.load_full_precision(_self, tmp.data)
            w.weight_loader = nv_loader
        elif w.dtype == torch.float8_e4m3fn:
            def f8_loader(param, tensor, shard_id, _l=loader):
                if tensor.dtype == torch.float8_e4m3fn:
                    view = nn.Parameter(param.data.view(torch.uint8), requires_grad=False)
                    _l(view, tensor.view(torch.uint8), shard_id)
                else:
                    raise TypeError("fp8 layer fed a non-fp8 tensor; quantise the checkpoint or drop the quant plan")
            w.weight_loader = f8_loader
        else:
            w.weight_loader = loader

    def _wire_scales(self, base: str) -> None:
        for name in ("weight_scale", "input_scale", "weight_global_scale"):
            p = getattr(self, name, None)
            if isinstance(p, nn.Parameter):
                p.hf_keys = {f"{base}.{name}": None}
                p.optional = True

                def scale_loader(param, tensor, shard_id=None):
                    t = tensor.reshape(-1) if tensor.dim() == 0 else tensor
                    if param.shape != t.shape:
                        param.data = t.to(dtype=param.dtype, device=param.device).clone()
                    else:
                        param.data.copy_(t.to(param.dtype))
                p.weight_loader = scale_loader

    def post_load(self) -> None:
        self.spec.process_after_loading(self)

    def _apply(self, x: torch.Tensor, n_local: int, k_local: int, bias: torch.Tensor | None) -> torch.Tensor:
        m = x.numel() // max(x.shape[-1], 1)
        kernel = get_linear_dispatcher().select(
            spec_id=self.spec.spec_id, M=m, N=n_local, K=k_local, in_dtype=x.dtype, out_dtype=self.params_dtype,
            device_type=x.device.type, capturing=pstate.current_mode() is P.Mode.GRAPH_CAPTURING)
        return kernel.apply(self, x, bias)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, spec={self.spec.spec_id}, bias={self.bias is not None}"


class ReplicatedLinear(LinearBase):
    def __init__(self, in_features: int, out_features: int, **kw) -> None:
        super().__init__(in_features, out_features, **kw)
        self._allocate(out_features, in_features)
        base = self.prefix
        if base:
            self._wire_weight({f"{base}.weight": None}, shards.replicated())
            if self.bias is not None:
                self.bias.hf_keys = {f"{base}.bias": None}
            self._wire_scales(base)

    def forward(self, x: torch.Tensor):
        b = None if self.skip_bias_add else self.bias
        return self._apply(x, self.out_features, self.in_features, b), (self.bias if self.skip_bias_add else None)


class ColumnParallelLinear(LinearBase):
    def __init__(self, in_features: int, out_features: int, *, axis: str = "tp", sp_axis: str | None = None,
                 gather_output: bool = False, mesh=None, _defer: bool = False, **kw) -> None:
        super().__init__(in_features, out_features, **kw)
        mesh = mesh if mesh is not None else pstate.default_mesh()
        self.axis, self.sp_axis, self.gather_output, self.mesh = axis, sp_axis, gather_output, mesh
        self.tp_rank, self.tp_size = _axis_info(axis, mesh)
        if out_features % self.tp_size:
            raise ValueError(f"out_features={out_features} is not divisible by {axis} size {self.tp_size}")
        self.output_size_per_partition = out_features // self.tp_size
        self.input_size_per_partition = in_features
        if _defer:
            return
        self._allocate(self.output_size_per_partition, in_features)
        base = self.prefix
        if base:
            self._wire_weight({f"{base}.weight": None}, shards.sharded(0, axis, mesh),
                              {f"{base}.weight": (out_features, in_features)})
            if self.bias is not None:
                self.bias.hf_keys = {f"{base}.bias": None}
                self.bias.hf_shapes = {f"{base}.bias": (out_features,)}
                self.bias.weight_loader = shards.sharded(0, axis, mesh)
            self._wire_scales(base)

    def forward(self, x: torch.Tensor):
        if self.sp_axis is not None:
            x = P.all_gather(x, axis=self.sp_axis, dim=0, mesh=self.mesh)
        b = None if self.skip_bias_add else self.bias
        y = self._apply(x, self.output_size_per_partition, self.input_size_per_partition, b)
        if self.gather_output and self.tp_size > 1:
            y = P.all_gather(y, axis=self.axis, dim=-1, mesh=self.mesh)
        return y, (self.bias if self.skip_bias_add else None)


class MergedColumnParallelLinear(ColumnParallelLinear):
    """``output_sizes`` projections sharing one input, stored as one weight.

    ``interleave=True`` (two equal legs) stores rows alternately (gate0, up0, gate1, ...),
    the layout the GEMM's gated-activation epilogue consumes.
    """

    DEFAULT_HF_LEGS: tuple[str, ...] = ("gate_proj", "up_proj")

    def __init__(self, in_features: int, output_sizes: Sequence[int], *, hf_legs: Sequence[str] | None = None,
                 interleave: bool = False, **kw) -> None:
        super().__init__(in_features, sum(output_sizes), _defer=True, **kw)
        self.output_sizes = tuple(output_sizes)
        self.interleave = interleave
        legs = tuple(hf_legs) if hf_legs is not None else self.DEFAULT_HF_LEGS
        if len(legs) != len(self.output_sizes):
            raise ValueError("hf_legs and output_sizes differ in length")
        if interleave and len(set(self.output_sizes)) != 1:
            raise ValueError("interleave needs equally sized legs")
        for s in self.output_sizes:
            if s % self.tp_size:
                raise ValueError(f"leg of size {s} is not divisible by {self.axis} size {self.tp_size}")
        self.hf_legs = legs
        local = [s // self.tp_size for s in self.output_sizes]
        self._allocate(sum(local), in_features)
        parent = self.prefix.rsplit(".", 1)[0] if "." in self.prefix else ""
        self.leg_prefixes = tuple(f"{parent}.{leg}" if parent else leg for leg in legs)
        table, off = {}, 0
        for i, n in enumerate(local):
            table[i] = (off, n)
            off += n
        if self.prefix:
            keys = {f"{lp}.weight": i for i, lp in enumerate(self.leg_prefixes)}
            shapes = {f"{lp}.weight": (self.output_sizes[i], in_features) for i, lp in enumerate(self.leg_prefixes)}
            self._wire_weight(keys, shards.fused(0, table, self.axis, self.mesh, interleave=interleave), shapes)
            if self.bias is not None:
                self.bias.hf_keys = {f"{lp}.bias": i for i, lp in enumerate(self.leg_prefixes)}
                self.bias.hf_shapes = {f"{lp}.bias": (self.output_sizes[i],) for i, lp in enumerate(self.leg_prefixes)}
                self.bias.weight_loader = shards.fused(0, table, self.axis, self.mesh, interleave=interleave)


class QKVParallelLinear(ColumnParallelLinear):
    """Fused q/k/v projection. Local layout: ``[q heads | k heads | v heads]``."""

    DEFAULT_HF_LEGS: tuple[str, ...] = ("q_proj", "k_proj", "v_proj")

    def __init__(self, hidden_size: int, head_dim: int, total_num_heads: int, total_num_kv_heads: int | None = None, *,
                 hf_legs: Sequence[str] | None = None, **kw) -> None:
        kvh = total_num_kv_heads if total_num_kv_heads is not None else total_num_heads
        axis, mesh = kw.get("axis", "tp"), kw.get("mesh")
        mesh = mesh if mesh is not None else pstate.default_mesh()
        _, tp = _axis_info(axis, mesh)
        if total_num_heads % tp:
            raise ValueError(f"num_heads={total_num_heads} is not divisible by {axis} size {tp}")
        if kvh >= tp:
            if kvh % tp:
                raise ValueError(f"num_kv_heads={kvh} is not divisible by {axis} size {tp}")
            kv_local, kv_rep = kvh // tp, 1
        else:
            if tp % kvh:
                raise ValueError(f"{axis} size {tp} is not a multiple of num_kv_heads={kvh}")
            kv_local, kv_rep = 1, tp // kvh
        q_local = total_num_heads // tp
        full_out = (total_num_heads + 2 * kvh) * head_dim
        # out_features of the base class must divide by tp; the replicated-KV case does not, so bypass
        LinearBase.__init__(self, hidden_size, full_out, **{k: v for k, v in kw.items() if k not in ("axis", "mesh", "sp_axis", "gather_output")})
        self.axis, self.mesh = axis, mesh
        self.sp_axis, self.gather_output = kw.get("sp_axis"), False
        self.tp_rank, self.tp_size = _axis_info(axis, mesh)
        self.head_dim, self.total_num_heads, self.total_num_kv_heads = head_dim, total_num_heads, kvh
        self.num_heads, self.num_kv_heads, self.num_kv_head_replicas = q_local, kv_local, kv_rep
        self.q_size, self.kv_size = q_local * head_dim, kv_local * head_dim
        self.output_size_per_partition = self.q_size + 2 * self.kv_size
        self.input_size_per_partition = hidden_size
        self.hf_legs = tuple(hf_legs) if hf_legs is not None else self.DEFAULT_HF_LEGS
        self._allocate(self.output_size_per_partition, hidden_size)
        parent = self.prefix.rsplit(".", 1)[0] if "." in self.prefix else ""
        self.leg_prefixes = tuple(f"{parent}.{leg}" if parent else leg for leg in self.hf_legs)
        table = {"q": (0, self.q_size), "k": (self.q_size, self.kv_size), "v": (self.q_size + self.kv_size, self.kv_size)}
        rep = {"q": 1, "k": kv_rep, "v": kv_rep}
        full = {"q": total_num_heads * head_dim, "k": kvh * head_dim, "v": kvh * head_dim}
        if self.prefix:
            ids = ("q", "k", "v")
            keys = {f"{lp}.weight": ids[i] for i, lp in enumerate(self.leg_prefixes)}
            shapes = {f"{lp}.weight": (full[ids[i]], hidden_size) for i, lp in enumerate(self.leg_prefixes)}
            self._wire_weight(keys, shards.fused(0, table, axis, mesh, replicate=rep), shapes)
            if self.bias is not None:
                self.bias.hf_keys = {f"{lp}.bias": ids[i] for i, lp in enumerate(self.leg_prefixes)}
                self.bias.hf_shapes = {f"{lp}.bias": (full[ids[i]],) for i, lp in enumerate(self.leg_prefixes)}
                self.bias.weight_loader = shards.fused(0, table, axis, mesh, replicate=rep)


class RowParallelLinear(LinearBase):
    def __init__(self, in_features: int, out_features: int, *, axis: str = "tp", sp_axis: str | None = None,
                 input_is_parallel: bool = True, reduce_results: bool = True, mesh=None, **kw) -> None:
        super().__init__(in_features, out_features, **kw)
        mesh = mesh if mesh is not None else pstate.default_mesh()
        self.axis, self.sp_axis, self.mesh = axis, sp_axis, mesh
        self.input_is_parallel, self.reduce_results = input_is_parallel, reduce_results
        self.tp_rank, self.tp_size = _axis_info(axis, mesh)
        if in_features % self.tp_size:
            raise ValueError(f"in_features={in_features} is not divisible by {axis} size {self.tp_size}")
        self.input_size_per_partition = in_features // self.tp_size
        self.output_size_per_partition = out_features
        self._allocate(out_features, self.input_size_per_partition)
        base = self.prefix
        if base:
            self._wire_weight({f"{base}.weight": None}, shards.sharded(1, axis, mesh),
                              {f"{base}.weight": (out_features, in_features)})
            if self.bias is not None:
                self.bias.hf_keys = {f"{base}.bias": None}
            self._wire_scales(base)

    def forward(self, x: torch.Tensor):
        if not self.input_is_parallel and self.tp_size > 1:
            x = x.chunk(self.tp_size, dim=-1)[self.tp_rank].contiguous()
        # the bias joins the sum exactly once: on rank 0 before the reduction
        fuse_bias = self.bias is not None and not self.skip_bias_add and self.tp_rank == 0
        y = self._apply(x, self.out_features, self.input_size_per_partition, self.bias if fuse_bias else None)
        if self.tp_size > 1:
            if self.sp_axis is not None:
                y = P.reduce_scatter(y, axis=self.sp_axis, dim=0, mesh=self.mesh)
            elif self.reduce_results:
                y = P.all_reduce(y, axis=self.axis, mesh=self.mesh)
        return y, (self.bias if self.skip_bias_add else None)


__all__ = ["LinearBase", "ReplicatedLinear", "ColumnParallelLinear", "MergedColumnParallelLinear",
           "QKVParallelLinear", "RowParallelLinear"]
