"""Data-parallel Pi0.5: every GPU holds a full replica and serves ``per_rank_B`` robots.

Rank 0 is the router: it pads the request to ``dp * per_rank_B`` rows and sends each
peer its shard over NCCL point-to-point; every rank runs the single-GPU scheduler; the
action chunks are gathered over the ``dp`` axis. Against the reference's router
(phyai/src/phyai/models/pi05/scheduler_wn_pi05.py:62-191):

* the four per-peer sends are one grouped p2p launch, and rank 0 does not wait for it: its own
  vision stage starts while the shards are still on the wire (the send buffers are kept until the
  next step);
* there is no header exchange and no host sync in front of the step. A request rank 0 cannot
  serve still reaches the peers, as a shard whose prompt lengths are -1, so every rank raises
  instead of leaving the peers blocked in a receive (the reference documents that hang);
* on CUDA the 3 KB action chunks go back through peer memory (one kernel that stores into every
  rank's buffer) instead of an NCCL all-gather; ``PHYAI_PEER_COMM=0`` keeps NCCL.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ... import parallel as P
from ...env import envs
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
        self._peer = None                     # PeerStream for the chunk gather; False = NCCL
        self._inflight: tuple[list, list] = ([], [])

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

    LENS_SLOT = 2          # position of ``lang_lens`` in ``_pack`` / ``_shapes``

    def _gather(self, local: torch.Tensor) -> torch.Tensor:
        """Action chunks of every rank, in rank order, on every rank."""
        if self._peer is None and local.is_cuda and envs.PHYAI_PEER_COMM.get() and local.dtype == torch.bfloat16 \
                and local[0].numel() % 8 == 0:
            try:
                from ...parallel.symm import PeerGroup

                pg = PeerGroup.for_axis(self.mesh, "dp")
                self._peer = pg.stream("dp:chunks", local.shape[0], local[0].numel())
            except Exception as e:  # noqa: BLE001 - NCCL serves the gather instead
                import logging

                logging.getLogger(__name__).warning("dp gather over peer memory unavailable (%s): using NCCL", e)
                self._peer = False
            ok = torch.tensor([1 if self._peer else 0], dtype=torch.int32, device=local.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.mesh.axis_group("dp"))   # all ranks take the same path
            if int(ok.item()) == 0:
                self._peer = False
        if self._peer:
            rows = self._peer.all_gather_rows(local.reshape(local.shape[0], -1).contiguous())
            return rows.view(self.dp_size * local.shape[0], *local.shape[1:])
        if self._peer is None:
            self._peer = False
        return P.all_gather(local.contiguous(), axis="dp", dim=0, mesh=self.mesh)

    @torch.no_grad()
    def step(self, request: PI05Request | None) -> torch.Tensor:
        if self.dp_size == 1:
            return self.local.step(request)
        R, N, pr, dev, dt = self.dp_rank, self.dp_size, self.per_rank_B, self.device, self.dtype
        group = self.mesh.axis_group("dp")
        ranks = self.mesh.axis_ranks("dp")
        on_gpu = dev.type == "cuda"
        if R == 0:
            for w in self._inflight[0]:          # last step's sends: long done, this only releases their buffers
                w.wait()
            self._inflight = ([], [])
            err: Exception | None = None
            real_B, total = 0, N * pr
            try:
                real_B = int(request.pixel_values.shape[0])
                if real_B > total:
                    raise ValueError(f"batch {real_B} exceeds DP capacity dp_size*per_rank_B={total}")
                full = [_pad_rows(t, total) for t in self._pack(request, real_B)]
            except Exception as e:  # noqa: BLE001 - the peers learn of it through a poisoned shard
                err = e
                full = [torch.zeros((total, *shape[1:]), dtype=dt if kind is None else kind, device=dev)
                        for shape, kind in self._shapes()]
                full[self.LENS_SLOT].fill_(-1)
            ops_ = [dist.P2POp(dist.isend, t[r * pr:(r + 1) * pr].contiguous(), ranks[r], group)
                    for r in range(1, N) for t in full]
            works = dist.batch_isend_irecv(ops_)
            if on_gpu:
                self._inflight = (works, [o.tensor for o in ops_])    # rank 0 computes while the shards travel
            else:
                for w in works:
                    w.wait()
            if err is not None:
                raise err
            shard = self._unpack([t[:pr] for t in full])
        else:
            bufs = [torch.empty(shape, dtype=dt if kind is None else kind, device=dev) for shape, kind in self._shapes()]
            for w in dist.batch_isend_irecv([dist.P2POp(dist.irecv, b, ranks[0], group) for b in bufs]):
                w.wait()
            if int(bufs[self.LENS_SLOT].min()) < 0:
                raise RuntimeError("rank 0 rejected the request")
            shard = self._unpack(bufs)
        # rows past real_B are padding: give them an empty prompt so they cost the smallest bucket
        local = self.local.step(shard)
        gathered = self._gather(local)
        return gathered[:real_B].clone() if R == 0 else gathered

    def close(self) -> None:
        self.local.close()


__all__ = ["PI05WNScheduler"]
