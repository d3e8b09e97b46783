"""Weight-loader factories: how one checkpoint tensor lands in one parameter.

A loader has the signature ``loader(param, tensor, shard_id)`` and copies the part
of ``tensor`` this rank owns into ``param``. Factories (reference:
phyai/src/phyai/weights/shards.py:23-158):

* ``replicated``      whole tensor on every rank
* ``sharded``         slice one dim by the rank's position on a mesh axis
* ``fused``           several checkpoint tensors ("legs") stacked along one dim of
                      one parameter, each leg sliced per rank (QKV, gate/up),
                      optionally row-interleaved
* ``vocab``           dim-0 slice of a vocabulary padded to a multiple, zero tail
* ``weight_norm_fold`` ``g * v / ||v||`` folded into a plain weight
"""

from __future__ import annotations

from typing import Callable, Mapping, Sequence

import torch

Loader = Callable[[torch.nn.Parameter, torch.Tensor, object], None]


def _axis_pos(axis: str | None, mesh) -> tuple[int, int]:
    if axis is None:
        return 0, 1
    if mesh is None:
        from ..parallel import state

        mesh = state.default_mesh()
    if mesh is None:
        return 0, 1
    return mesh.axis_local_rank(axis), mesh.axis_size(axis)


def _pin(mesh):
    """The mesh a loader works on is the one active when its layer was built, not when weights arrive."""
    if mesh is not None:
        return mesh
    from ..parallel import state

    return state.default_mesh()


def _copy(param: torch.nn.Parameter, src: torch.Tensor, dst_view: torch.Tensor | None = None) -> None:
    dst = param.data if dst_view is None else dst_view
    if dst.shape != src.shape:
        raise ValueError(f"shape mismatch: parameter slice {tuple(dst.shape)} vs checkpoint {tuple(src.shape)}")
    dst.copy_(src.to(dtype=dst.dtype))


def replicated() -> Loader:
    def load(param, tensor, shard_id=None):
        _copy(param, tensor)
    return load


def sharded(dim: int, axis: str | None = "tp", mesh=None, *, replicate: int = 1) -> Loader:
    """Slice ``dim`` into ``size/replicate`` parts; ``replicate`` consecutive ranks share a part."""
    mesh = _pin(mesh)

    def load(param, tensor, shard_id=None):
        r, n = _axis_pos(axis, mesh)
        parts = max(n // max(replicate, 1), 1)
        idx = r // max(replicate, 1)
        if tensor.shape[dim] % parts:
            raise ValueError(f"dim {dim} of size {tensor.shape[dim]} is not divisible into {parts} shards")
        step = tensor.shape[dim] // parts
        _copy(param, tensor.narrow(dim, idx * step, step))
    return load


def fused(fuse_dim: int, legs: Mapping[object, tuple[int, int]] | Sequence[tuple[object, int, int]],
          axis: str | None = "tp", mesh=None, *, replicate: Mapping[object, int] | None = None,
          interleave: bool = False) -> Loader:
    """``legs``: shard_id -> (offset, size) inside the *local* parameter along ``fuse_dim``.

    Each checkpoint leg is sliced for this rank (``replicate[shard_id]`` ranks share a
    slice: KV heads replicated when tp > kv_heads) and copied at its offset. With
    ``interleave`` and two equal legs, leg 0 fills even rows and leg 1 odd rows (the
    layout the gated-activation GEMM epilogue reads).
    """
    table = dict(legs) if isinstance(legs, Mapping) else {k: (o, s) for k, o, s in legs}
    order = list(table.keys())
    mesh = _pin(mesh)

    def load(param, tensor, shard_id=None):
        if shard_id not in table:
            raise KeyError(f"unknown shard id {shard_id!r}; expected one of {order}")
        off, size = table[shard_id]
        r, n = _axis_pos(axis, mesh)
        rep = (replicate or {}).get(shard_id, 1)
        parts = max(n // max(rep, 1), 1)
        idx = r // max(rep, 1)
        if tensor.shape[fuse_dim] % parts:
            raise ValueError(f"leg {shard_id!r}: dim {fuse_dim} of {tensor.shape[fuse_dim]} not divisible by {parts}")
        step = tensor.shape[fuse_dim] // parts
        src = tensor.narrow(fuse_dim, idx * step, step)
        if step != size:
            raise ValueError(f"leg {shard_id!r}: local size {step} != declared {size}")
        if interleave:
            pos = order.index(shard_id)
            view = param.data.movedim(fuse_dim, 0)
            view[pos::len(order)].copy_(src.movedim(fuse_dim, 0).to(view.dtype))
        else:
            _copy(param, src, param.data.narrow(fuse_dim, off, size))
    return load


def vocab(padded_size: int, axis: str | None = "tp", mesh=None) -> Loader:
    """Rows ``[r*per, (r+1)*per)`` of the padded vocabulary; rows past the real vocab are zero."""
    mesh = _pin(mesh)

    def load(param, tensor, shard_id=None):
        r, n = _axis_pos(axis, mesh)
        per = padded_size // n
        lo, hi = r * per, min((r + 1) * per, tensor.shape[0])
        param.data.zero_()
        if hi > lo:
            param.data[: hi - lo].copy_(tensor[lo:hi].to(param.dtype))
    return load


def weight_norm_fold(dim: int = 0) -> Loader:
    """Legs ``"g"`` and ``"v"`` of a weight-normed layer -> ``w = g * v / ||v||`` (norm over all dims but ``dim``)."""
    stash: dict[int, dict[str, torch.Tensor]] = {}

    def load(param, tensor, shard_id=None):
        slot = stash.setdefault(id(param), {})
        slot[str(shard_id)] = tensor.float()
        if "g" in slot and "v" in slot:
            v, g = slot["v"], slot["g"]
            dims = [d for d in range(v.dim()) if d != dim]
            w = g * v / v.norm(dim=dims, keepdim=True).clamp_min(1e-12)
            _copy(param, w)
            stash.pop(id(param), None)
    return load


__all__ = ["replicated", "sharded", "fused", "vocab", "weight_norm_fold", "Loader"]
