"""Data-parallel Pi0.5: every GPU holds a full replica and serves ``per_rank_B`` robots.

Rank 0 is the router: it pads the request to ``dp * per_rank_B`` rows and sends each
peer its shard over NCCL point-to-point; every rank runs the single-GPU scheduler; the
action chunks are all-gathered over the ``dp`` axis. The four per-peer sends of the
reference (phyai/src/phyai/models/pi05/scheduler_wn_pi05.py:62-191) are batched into one
grouped p2p launch per step, and a header broadcast tells the peers whether rank 0
accepted the request, so an oversize batch raises on every rank instead of leaving the
peers blocked in a receive.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ... import parallel as P
from ...runtime import Scheduler
from .scheduler_ws1_pi05 import PI05Request, PI05WS1Scheduler


def _pad_rows(t: torch.Tensor, rows: int) -> torch.Tensor:
    if t.shape[0] == rows:
        return t
    out = torch.zeros((rows, *t.shape[1:]), dtype=t.dtype, device=t.device)
    out[: t.shape[0]] = t
    return out


class PI05WNScheduler(Scheduler):
    def __init__(self, local: PI05WS1Scheduler, *, device: torch.device | str | None = None) -> None:
        self.local = local
        self.device = torch.device(device) if device is not None else local.device
        self.dtype, self.cfg = local.params_dtype, local.cfg
        self.num_images, self.per_rank_B = local.num_images, local.max_batch_size
        mesh = P.default_mesh()
        self.mesh = mesh
        self.dp_rank = mesh.axis_local_rank("dp") if mesh is not None else 0
        self.dp_size = mesh.axis_size("dp") if mesh is not None else 1

    def setup(self) -> None:
        if self.dp_size > 1 and self.mesh.world_size != self.dp_size:
            raise RuntimeError(f"pi05_wn is pure data parallelism: dp_size={self.dp_size} must equal "
                               f"world_size={self.mesh.world_size}")
        self.local.setup()

    # ---- what travels: subclasses for other request types override these three
    def _shapes(self):
        """Per-rank shard shapes and dtypes (None = the parameter dtype), in the order of ``_pack``."""
        cfg, pr = self.cfg, self.per_rank_B
        v = cfg.vision
        return [((pr, self.num_images, v.num_channels, v.image_size, v.image_size), None), ((pr, cfg.tokenizer_max_length), torch.int64),
                ((pr,), torch.int64), ((pr, cfg.chunk_size, cfg.max_action_dim), None)]

    def _pack(self, request, real_B: int) -> list[torch.Tensor]:
        dev, dt = self.device, self.dtype
        nz = request.noise.to(dev, dt) if request.noise is not None else torch.randn(
            real_B, self.cfg.chunk_size, self.cfg.max_action_dim, device=dev, dtype=dt)
        return [request.pixel_values.to(dev, dt), request.input_ids.to(dev, torch.int64), request.lang_lens.to(dev, torch.int64), nz]

    def _unpack(self, tensors: list[torch.Tensor]):
        return PI05Request(*tensors)

    @torch.no_grad()
    def step(self, request: PI05Request | None) -> torch.Tensor:
        if self.dp_size == 1:
            return self.local.step(request)
        R, N, pr, dev, dt = self.dp_rank, self.dp_size, self.per_rank_B, self.device, self.dtype
        group = self.mesh.axis_group("dp")
        ranks = self.mesh.axis_ranks("dp")
        # header: [accepted, real_B]
        head = torch.zeros(2, dtype=torch.int64, device=dev)
        err: Exception | None = None
        if R == 0:
            try:
                real_B = int(request.pixel_values.shape[0])
                if real_B > N * pr:
                    raise ValueError(f"batch {real_B} exceeds DP capacity dp_size*per_rank_B={N * pr}")
                head[0], head[1] = 1, real_B
            except Exception as e:  # noqa: BLE001 - forwarded to every rank below
                err = e
        dist.broadcast(head, src=ranks[0], group=group)
        if int(head[0]) != 1:
            raise err if err is not None else RuntimeError("rank 0 rejected the request")
        real_B = int(head[1])
        if R == 0:
            total = N * pr
            full = [_pad_rows(t, total) for t in self._pack(request, real_B)]
            ops_ = []
            for r in range(1, N):
                for t in full:
                    ops_.append(dist.P2POp(dist.isend, t[r * pr:(r + 1) * pr].contiguous(), ranks[r], group))
            for w in dist.batch_isend_irecv(ops_):
                w.wait()
            shard = self._unpack([t[:pr] for t in full])
        else:
            bufs = [torch.empty(shape, dtype=dt if kind is None else kind, device=dev) for shape, kind in self._shapes()]
            for w in dist.batch_isend_irecv([dist.P2POp(dist.irecv, b, ranks[0], group) for b in bufs]):
                w.wait()
            shard = self._unpack(bufs)
        # rows past real_B are padding: give them an empty prompt so they cost the smallest bucket
        local = self.local.step(shard)
        gathered = P.all_gather(local.contiguous(), axis="dp", dim=0, mesh=self.mesh)
        return gathered[:real_B].clone() if R == 0 else gathered

    def close(self) -> None:
        self.local.close()


__all__ = ["PI05WNScheduler"]
