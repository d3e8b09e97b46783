"""``torch.distributed`` backends: NCCL for CUDA tensors, gloo for CPU tensors.

All ops are out-of-place at this level (``execute`` returns a new tensor). NCCL
collectives enqueue on the current stream and are capturable once the
communicator is warm; gloo is host-side and never capturable. Reference:
phyai/src/phyai/parallel/backends/{torch_dist,gloo,pynccl}.py.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from ..backend import Call, Op

_REDUCE = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
           "avg": dist.ReduceOp.AVG, "prod": dist.ReduceOp.PRODUCT}


class _TorchDistBackend:
    name = "torch"
    device_type = "cpu"
    capturable = False

    def can_handle(self, call: Call) -> bool:
        return call.device_type == self.device_type and call.mesh.axis_size(call.axis) > 1

    def supports_capture(self) -> bool:
        return self.capturable

    # ------------------------------------------------------------------ ops
    def execute(self, call: Call, *tensors: torch.Tensor, **kw: Any):
        group = call.mesh.axis_group(call.axis)
        n = call.mesh.axis_size(call.axis)
        ranks = call.mesh.axis_ranks(call.axis)
        op = call.op
        if op is Op.ALL_REDUCE:
            out = tensors[0].clone()
            dist.all_reduce(out, op=_REDUCE[kw.get("reduce", "sum")], group=group)
            return out
        if op is Op.ALL_GATHER:
            x = tensors[0]
            dim = kw.get("dim", 0) % max(x.dim(), 1)
            xm = x.movedim(dim, 0).contiguous()
            out = torch.empty((n * xm.shape[0], *xm.shape[1:]), dtype=x.dtype, device=x.device)
            self._all_gather_into(out, xm, group, n)
            return out.movedim(0, dim) if dim else out
        if op is Op.REDUCE_SCATTER:
            x = tensors[0]
            dim = kw.get("dim", 0) % max(x.dim(), 1)
            xm = x.movedim(dim, 0).contiguous()
            if xm.shape[0] % n:
                raise ValueError(f"reduce_scatter: dim {dim} of size {xm.shape[0]} is not divisible by {n}")
            out = torch.empty((xm.shape[0] // n, *xm.shape[1:]), dtype=x.dtype, device=x.device)
            self._reduce_scatter_into(out, xm, group, n, _REDUCE[kw.get("reduce", "sum")])
            return out.movedim(0, dim) if dim else out
        if op is Op.ALL_TO_ALL:
            x = tensors[0]
            sd, cd = kw.get("split_dim", 0), kw.get("concat_dim", 0)
            parts = [p.contiguous() for p in x.chunk(n, dim=sd)]
            outs = [torch.empty_like(parts[0]) for _ in range(n)]
            dist.all_to_all(outs, parts, group=group)
            return torch.cat(outs, dim=cd)
        if op is Op.BROADCAST:
            out = tensors[0].clone()
            dist.broadcast(out, src=ranks[kw.get("src", 0)], group=group)
            return out
        if op is Op.SEND:
            dist.send(tensors[0].contiguous(), dst=ranks[kw["dst"]], group=group)
            return None
        if op is Op.RECV:
            dist.recv(tensors[0], src=ranks[kw["src"]], group=group)
            return tensors[0]
        if op is Op.BARRIER:
            dist.barrier(group=group)
            return None
        raise NotImplementedError(op)

    def _all_gather_into(self, out, x, group, n):
        dist.all_gather_into_tensor(out, x, group=group)

    def _reduce_scatter_into(self, out, x, group, n, rop):
        dist.reduce_scatter_tensor(out, x, op=rop, group=group)


class NcclBackend(_TorchDistBackend):
    name = "nccl"
    device_type = "cuda"
    capturable = True

    def execute(self, call: Call, *tensors: torch.Tensor, **kw: Any):
        if call.op is Op.ALL_TO_ALL:
            x = tensors[0]
            n = call.mesh.axis_size(call.axis)
            sd, cd = kw.get("split_dim", 0), kw.get("concat_dim", 0)
            xm = torch.cat([p.unsqueeze(0) for p in x.chunk(n, dim=sd)], 0).contiguous()
            out = torch.empty_like(xm)
            dist.all_to_all_single(out, xm, group=call.mesh.axis_group(call.axis))
            return torch.cat(list(out.unbind(0)), dim=cd)
        return super().execute(call, *tensors, **kw)


class GlooBackend(_TorchDistBackend):
    name = "gloo"
    device_type = "cpu"
    capturable = False

    def execute(self, call: Call, *tensors: torch.Tensor, **kw: Any):
        if call.op is Op.ALL_TO_ALL:
            # gloo has no all-to-all: gather everything and keep the pieces addressed to this rank
            x = tensors[0]
            group, n = call.mesh.axis_group(call.axis), call.mesh.axis_size(call.axis)
            sd, cd = kw.get("split_dim", 0), kw.get("concat_dim", 0)
            mine = torch.stack([p.contiguous() for p in x.chunk(n, dim=sd)])
            everyone = [torch.empty_like(mine) for _ in range(n)]
            dist.all_gather(everyone, mine, group=group)
            r = dist.get_rank(group)
            return torch.cat([e[r] for e in everyone], dim=cd)
        return super().execute(call, *tensors, **kw)

    def _all_gather_into(self, out, x, group, n):
        parts = list(out.chunk(n, dim=0))
        dist.all_gather(parts, x, group=group)

    def _reduce_scatter_into(self, out, x, group, n, rop):
        # gloo has no reduce_scatter: all-reduce then keep this rank's slice
        full = x.clone()
        dist.all_reduce(full, op=rop, group=group)
        r = dist.get_rank(group)
        out.copy_(full.chunk(n, dim=0)[r])


__all__ = ["NcclBackend", "GlooBackend"]
