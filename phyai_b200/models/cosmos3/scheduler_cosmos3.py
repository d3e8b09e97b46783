"""Cosmos3 denoising schedulers: text/image-to-video [+ sound] and the three action modes.

One implementation serves every world size. With a ``cfg`` mesh axis of size 2 the two
guidance branches run on different GPU groups (``cfg`` rank 0 = conditional, 1 =
unconditional) and the guided velocity is formed by the peer-memory CFG exchange kernel
(each rank writes its velocity into the partner's buffer and applies
``uncond + g (cond - uncond)`` in the same kernel) or, where that path is unavailable, by an
all-gather over ``cfg``. With one rank per branch pair the branches run back to back. The
transformer itself may be tensor parallel over ``tp``.

On one GPU the branch passes of a denoise step are a CUDA graph kept per request geometry (:class:`LoopSlot`,
:class:`StepGraph`): the first step of the first request of a geometry runs launch by launch (it builds the
workspaces and K/V buffers), the second is captured, and every later step, of that request and of the following
ones, replays it. What changes between steps or requests stays outside the graph or in buffers it reads: the
timestep in a one-element device buffer, the latents, masks and domain ids in tensors of the slot that a request
copies its values into, the prompt in the slot's conditions (text K/V and rotary table overwritten in place), the
sampler kernel (its coefficients are launch arguments) after every replay. The reference issues every step
eagerly (phyai/src/phyai/models/cosmos3/scheduler_ws1_cosmos3_policy.py:102-106 notes graph capture as open).

Reference: phyai/src/phyai/models/cosmos3/scheduler_ws1_cosmos3.py:29-320,
scheduler_wn_cosmos3.py:54-317, scheduler_ws1_cosmos3_policy.py:25-279,
scheduler_wn_cosmos3_policy.py:50-303.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import numpy as np
import torch

from ... import ops
from ... import parallel as P
from ...env import envs
from ...runtime import Scheduler
from ...runtime.cuda_graph_manager import CudaGraph
from ...utils.profile import event_scope
from .modeling_cosmos3 import Cosmos3Condition
from .sampler_unipc import FusedUniPCStream, UniPCMultistepSampler
from .transformer_cosmos3 import Cosmos3Transformer


@dataclass
class Cosmos3T2VRequest:
    """Already-tokenised request. ``video_shape`` is the latent grid (t, h, w)."""

    text_ids: torch.Tensor
    text_mask: torch.Tensor
    neg_text_ids: torch.Tensor
    neg_text_mask: torch.Tensor
    video_shape: tuple[int, int, int]
    fps: float = 24.0
    num_inference_steps: int = 35
    guidance_scale: float = 6.0
    noise: torch.Tensor | None = None
    seed: int = 42
    cond_latents: torch.Tensor | None = None
    cond_frame_indexes: tuple[int, ...] = ()
    sound_frames: int | None = None
    sound_dim: int = 64
    sound_latent_fps: float = 25.0


@dataclass
class Cosmos3ActionRequest:
    """``mode``: policy (frame 0 clean, actions generated), forward_dynamics (frame 0 and the actions
    clean, video generated) or inverse_dynamics (whole video clean, actions generated)."""

    text_ids: torch.Tensor
    text_mask: torch.Tensor
    neg_text_ids: torch.Tensor
    neg_text_mask: torch.Tensor
    video_shape: tuple[int, int, int]
    mode: str
    domain_id: int
    action_chunk: int
    raw_action_dim: int
    action_dim: int = 64
    cond_video_latents: torch.Tensor | None = None
    cond_video_pixels: torch.Tensor | None = None
    cond_action: torch.Tensor | None = None
    cond_frame_indexes: tuple[int, ...] | None = None
    fps: float = 24.0
    num_inference_steps: int = 30
    guidance_scale: float = 1.0
    seed: int = 42


ACTION_MODES = ("policy", "forward_dynamics", "inverse_dynamics")


def pixel_to_latent_shape(num_frames: int, height: int, width: int, *, temporal: int = 4, spatial: int = 16):
    return (num_frames - 1) // temporal + 1, height // spatial, width // spatial


def seeded_normal(shape, seed: int, device, dtype) -> torch.Tensor:
    """Identical noise on every rank: NumPy's legacy generator, as the reference uses."""
    return torch.from_numpy(np.random.RandomState(int(seed)).standard_normal(shape).astype("float32")).to(device, dtype)


class StepGraph:
    """The model passes of one denoise step, captured once and replayed.

    ``run(fn)``: the first call runs ``fn`` as it is (lazy state is built there), the second captures it into a
    CUDA graph and replays it, later calls only replay. ``fn`` must read everything that changes between steps
    from tensors whose storage stays put, and return tensors: they live in the graph's memory pool and are
    overwritten by the next replay. A capture that fails (an op that cannot be captured) turns the graph off
    for good and runs ``fn`` eagerly; nothing the capture issued has executed by then."""

    def __init__(self, enabled: bool) -> None:
        self.enabled = bool(enabled)
        self.graph: CudaGraph | None = None
        self.calls = self.replays = 0
        self.launches = 0        # kernels of this package in one replay (``ops.launch_counter`` sees the capture only)

    def run(self, fn):
        self.calls += 1
        if not self.enabled or self.calls == 1:
            return fn()
        if self.graph is None:
            graph = CudaGraph("cosmos3.step", warmup_iters=0)      # the eager first step was the warm-up
            before = ops.launch_counter()
            try:
                graph.capture(fn, {})
            except Exception as e:  # noqa: BLE001 - the request is served eagerly instead, and it is said out loud
                import logging

                logging.getLogger(__name__).warning("denoise step not captured (%s: %s): running it launch by launch",
                                                    type(e).__name__, e)
                self.enabled = False
                return fn()
            self.graph, self.launches = graph, ops.launch_counter() - before
        self.replays += 1
        return self.graph.replay()


@dataclass
class LoopSlot:
    """Device state of one request geometry that outlives the request, so that one captured step serves all of them:
    the tensors a step reads (latents, masks, timestep, domain ids), the conditions of the guidance branches with the
    buffers of the CUDA path inside them, and the graph."""

    graph: StepGraph
    tensors: dict[str, torch.Tensor] = dataclasses.field(default_factory=dict)
    conds: dict[str, Cosmos3Condition] = dataclasses.field(default_factory=dict)
    opened_at: tuple[int, bool] = (0, False)       # replays so far and "already captured" when the current request began

    @property
    def persistent(self) -> bool:
        return self.graph.enabled

    def hold(self, name: str, value: torch.Tensor | None) -> torch.Tensor | None:
        """The slot's tensor ``name`` with the values of ``value`` (a slot without a graph hands ``value`` through)."""
        if value is None or not self.persistent:
            return value
        cur = self.tensors.get(name)
        if cur is None:
            cur = self.tensors[name] = value.contiguous().clone()
        else:
            cur.copy_(value)
        return cur


def real_text_len(mask: torch.Tensor) -> int:
    """Longest unpadded prompt of a batch: the text rows a condition keeps."""
    return int(mask.sum(dim=1).max().item())


class Cosmos3Runner:
    """Holds the per-branch condition (encoded once per request) and runs the per-step GEN pass."""

    def __init__(self, transformer: Cosmos3Transformer) -> None:
        self.transformer = transformer
        self._cond: dict[str, Cosmos3Condition] = {}
        self._held: dict[str, Cosmos3Condition] | None = None

    def reset(self, held: dict[str, Cosmos3Condition] | None = None) -> None:
        """Forget the last request's prompts. ``held``: conditions that a captured step reads; a new prompt is written
        into them in place instead of replacing them."""
        self._cond.clear()
        self._held = held

    def prepare(self, branch: str, *, text_ids, text_mask, video_shape, fps, action_len: int = 0, sound_len: int = 0,
                sound_fps=None) -> Cosmos3Condition:
        c = self.transformer.encode_condition(text_ids, text_mask, video_shape, fps, action_len=action_len,
                                              sound_len=sound_len, sound_fps=sound_fps)
        if self._held is not None:
            kept = self._held.get(branch)
            if kept is None:
                self._held[branch] = c
            else:
                kept.refresh_from(c)
                c = kept
        self._cond[branch] = c
        return c

    def forward(self, branch: str, video, t, *, text_ids, text_mask, video_shape, fps, noisy_frame_mask=None,
                action_latents=None, action_domain_id=None, action_noisy_mask=None, sound_latents=None, sound_fps=None):
        c = self._cond.get(branch)
        if c is None:
            c = self.prepare(branch, text_ids=text_ids, text_mask=text_mask, video_shape=video_shape, fps=fps,
                             action_len=0 if action_latents is None else action_latents.shape[1],
                             sound_len=0 if sound_latents is None else sound_latents.shape[1], sound_fps=sound_fps)
        return self.transformer(video, t.expand(video.shape[0]), c, noisy_frame_mask=noisy_frame_mask,
                                action_latents=action_latents, action_domain_id=action_domain_id,
                                action_noisy_mask=action_noisy_mask, sound_latents=sound_latents)


class _GuidanceMixin:
    """CFG over one or two ``cfg`` ranks."""

    #: UniPC update, guidance combine and clean frames as one kernel per step on CUDA bf16 (PHYAI_COSMOS3_FUSED_SAMPLER=0: tensor ops)
    fused_sampler = bool(envs.PHYAI_COSMOS3_FUSED_SAMPLER.get())

    #: branch passes of a step as one CUDA graph per request geometry on a single GPU (PHYAI_COSMOS3_GRAPH=0: every launch from the host)
    graph_steps = bool(envs.PHYAI_COSMOS3_GRAPH.get())
    #: request geometries whose buffers and graph are kept (least recently used goes first)
    max_loop_slots = 2
    #: graph replays of the last request (0: it ran launch by launch), and how many kernels of this package those replays
    #: ran that ``ops.launch_counter`` did not see (it counts a capture once and no replay)
    last_graph_replays = 0
    last_graph_uncounted = 0

    def _graphable(self, fused: bool) -> bool:
        """Whether the steps of a request can be captured: the fused CUDA path of the transformer on one rank
        (tensor-parallel and two-rank guidance steps hold peer-memory collectives whose launch arguments change per
        call), the one-kernel sampler (the tensor-op one rebinds the latents), and graphs allowed by the engine."""
        from ...engine_config import get_engine_config

        tr = self.transformer
        return bool(self.graph_steps and fused and self.device.type == "cuda" and tr.use_fused and self.cfg_size == 1
                    and tr.gen_layers[0].mlp.down_proj.tp_size == 1 and get_engine_config().runtime.use_cuda_graph)

    def _loop_slot(self, signature: tuple, fused: bool) -> LoopSlot:
        """The kept slot of this request geometry where its steps can be captured, else a throw-away slot that keeps
        nothing."""
        tr = self.transformer
        if not self._graphable(fused):
            return LoopSlot(StepGraph(False))
        slots = self.__dict__.setdefault("_loop_slots", {})
        key = (signature, bool(tr.serve_fp8), bool(tr.serve_nvfp4))
        slot = slots.pop(key, None)
        if slot is None:
            slot = LoopSlot(StepGraph(True))
            while len(slots) >= self.max_loop_slots:
                slots.pop(next(iter(slots)))
        slots[key] = slot                      # most recently used last
        slot.opened_at = (slot.graph.replays, slot.graph.graph is not None)
        return slot

    def _close_slot(self, slot: LoopSlot) -> None:
        """Book-keeping after the loop of a request."""
        g = slot.graph
        replays0, captured0 = slot.opened_at
        self.last_graph_replays = g.replays - replays0
        captured_now = g.graph is not None and not captured0
        self.last_graph_uncounted = max(self.last_graph_replays - (1 if captured_now else 0), 0) * g.launches

    def drop_loop_slots(self) -> None:
        """Free the kept request geometries (their buffers and graphs)."""
        self.__dict__.pop("_loop_slots", None)

    def close(self) -> None:
        self.drop_loop_slots()
        super().close()

    def _init_guidance(self) -> None:
        mesh = P.default_mesh()
        self.mesh = mesh
        self.cfg_size = mesh.axis_size("cfg") if mesh is not None else 1
        self.cfg_rank = mesh.axis_local_rank("cfg") if mesh is not None else 0
        if self.cfg_size not in (1, 2):
            raise ValueError(f"cfg axis must have size 1 or 2, got {self.cfg_size}")
        self._peer = None

    def _peer_exchange(self):
        """The guidance pair's peer group, or None when it cannot be had. Opening it is a collective, so the two
        ranks agree on the outcome before either uses it: a rank whose mapping failed while its partner's
        succeeded would otherwise call NCCL against a partner that waits in the peer kernel."""
        if self._peer is None and self.cfg_size == 2 and self.device.type == "cuda":
            import logging

            import torch.distributed as dist

            pg = None
            try:
                from ...parallel.symm import PeerGroup

                pg = PeerGroup.for_axis(self.mesh, "cfg")
            except Exception as e:     # noqa: BLE001 - any failure means "use NCCL", but it is said out loud
                logging.getLogger(__name__).warning("cfg peer exchange unavailable on this rank: %s", e)
            ok = torch.tensor([1 if pg is not None else 0], dtype=torch.int32, device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.mesh.axis_group("cfg"))
            if int(ok.item()) == 1:
                self._peer = pg
            else:
                if pg is not None:
                    pg._closed = True      # the partner never opened its side: drop the handle without the collective close
                self._peer = False
        return self._peer or None

    def guided(self, run_branch, g: float, do_cfg: bool):
        """``run_branch(name)`` -> tuple of velocity tensors; returns the guided tuple on every rank."""
        if not do_cfg:
            return run_branch("cond")
        if self.cfg_size == 1:
            c, u = run_branch("cond"), run_branch("uncond")
            return tuple(self._combine_local(a, b, g) for a, b in zip(c, u))
        mine = run_branch("cond" if self.cfg_rank == 0 else "uncond")
        peer = self._peer_exchange()
        out = []
        for v in mine:
            if peer is not None and v.is_cuda and v.dtype == torch.bfloat16 and v.numel() % 8 == 0:
                out.append(peer.cfg_exchange(v.contiguous(), is_cond=self.cfg_rank == 0, g=g))
            else:
                pair = P.all_gather(v[None].contiguous(), axis="cfg", dim=0, mesh=self.mesh)
                out.append((pair[1].float() + g * (pair[0].float() - pair[1].float())).to(v.dtype))
        return tuple(out)

    def guided_pair(self, run_branch, g: float, do_cfg: bool):
        """As :meth:`guided`, for a consumer that can combine the two branches itself (the fused sampler kernel):
        returns ``(velocities, uncond velocities or None)``; the second is set only when both branches ran here."""
        if do_cfg and self.cfg_size == 1:
            return run_branch("cond"), run_branch("uncond")
        return self.guided(run_branch, g, do_cfg), None

    @staticmethod
    def _combine_local(c: torch.Tensor, u: torch.Tensor, g: float) -> torch.Tensor:
        if c.is_cuda and c.dtype == torch.bfloat16:
            return ops.cfg_combine(c.contiguous(), u.contiguous(), g)
        return (u.float() + g * (c.float() - u.float())).to(c.dtype)


class Cosmos3T2VScheduler(_GuidanceMixin, Scheduler):
    def __init__(self, transformer: Cosmos3Transformer, *, vae=None, avae=None, device=None, flow_shift: float = 1.0,
                 use_karras_sigmas: bool = True) -> None:
        self.transformer = transformer
        self.device = torch.device(device) if device is not None else next(transformer.parameters()).device
        self.dtype = transformer.params_dtype
        self.latent_channel = transformer.config.latent_channel
        self.runner = Cosmos3Runner(transformer)
        self.vae, self.avae = vae, avae
        self._flow_shift, self._karras = flow_shift, use_karras_sigmas
        self.unipc: UniPCMultistepSampler | None = None
        self._init_guidance()

    def setup(self) -> None:
        self.unipc = UniPCMultistepSampler(flow_shift=self._flow_shift, use_karras_sigmas=self._karras)

    def _new_sampler(self, n: int) -> UniPCMultistepSampler:
        s = UniPCMultistepSampler(flow_shift=self._flow_shift, use_karras_sigmas=self._karras)
        s.set_timesteps(n, device=self.device)
        return s

    @torch.no_grad()
    def step(self, request: Cosmos3T2VRequest):
        if self.unipc is None:
            raise RuntimeError("call setup() before step()")
        dev, dt = self.device, self.dtype
        t_lat, h_lat, w_lat = request.video_shape
        with_sound = request.sound_frames is not None
        video = (request.noise.to(dev, dt).clone() if request.noise is not None
                 else seeded_normal((1, self.latent_channel, t_lat, h_lat, w_lat), request.seed, dev, dt))
        sound = None
        if with_sound:
            sound = seeded_normal((request.sound_dim, request.sound_frames), request.seed, dev, dt).t()[None].contiguous()
        cond_idx = list(request.cond_frame_indexes)
        cond_latents, frame_mask = None, None
        if request.cond_latents is not None and cond_idx:
            cond_latents = request.cond_latents.to(dev, dt)
            video[:, :, cond_idx] = cond_latents[:, :, cond_idx]
            frame_mask = torch.ones(1, t_lat, dtype=torch.bool, device=dev)
            frame_mask[:, cond_idx] = False
        prompts = {"cond": (request.text_ids.to(dev), request.text_mask.to(dev)),
                   "uncond": (request.neg_text_ids.to(dev), request.neg_text_mask.to(dev))}
        do_cfg = request.guidance_scale > 1.0
        sfps = request.sound_latent_fps if with_sound else None
        uni_v = self._new_sampler(request.num_inference_steps)
        uni_s = self._new_sampler(request.num_inference_steps) if with_sound else None
        scope = "cosmos3.t2av_denoise_loop" if with_sound else "cosmos3.denoise_loop"
        fused = self.fused_sampler and FusedUniPCStream.usable(video)
        branches = ("cond", "uncond") if do_cfg else ("cond",)
        slot = self._loop_slot(("t2v", tuple(video.shape), None if sound is None else tuple(sound.shape), frame_mask is not None,
                                tuple(real_text_len(prompts[b][1]) for b in branches)), fused)
        self.runner.reset(slot.conds if slot.persistent else None)
        if slot.persistent:
            # a captured step reads the slot's tensors and conditions: this request's values go into them
            video, sound, frame_mask = slot.hold("video", video), slot.hold("sound", sound), slot.hold("frame_mask", frame_mask)
            for b in branches:
                self.runner.prepare(b, text_ids=prompts[b][0], text_mask=prompts[b][1], video_shape=request.video_shape,
                                    fps=request.fps, sound_len=0 if sound is None else sound.shape[1], sound_fps=sfps)
        fused_v = fused_s = None
        if fused:
            # one kernel per stream and step: guidance combine, UniPC update and the clean frames in one pass
            video = video.contiguous()
            keep = None if frame_mask is None else ~frame_mask
            fused_v = FusedUniPCStream(uni_v, video, view=(video.shape[1], t_lat, h_lat * w_lat), keep=keep,
                                       cond=cond_latents if keep is not None else None)
            if with_sound:
                fused_s = FusedUniPCStream(uni_s, sound)
        graph = slot.graph
        tval = slot.hold("tval", torch.empty(1, device=dev, dtype=dt))      # one buffer for all steps: a captured step reads it
        with event_scope(scope):
            for timestep in uni_v.timesteps:
                tval.copy_(timestep.reshape(1))

                def run(branch: str):
                    ids, mask = prompts[branch]
                    out = self.runner.forward(branch, video, tval, text_ids=ids, text_mask=mask,
                                              video_shape=request.video_shape, fps=request.fps, noisy_frame_mask=frame_mask,
                                              sound_latents=sound, sound_fps=sfps)
                    return out if with_sound else (out,)

                if fused_v is not None:
                    vel, unc = graph.run(lambda: self.guided_pair(run, request.guidance_scale, do_cfg))
                    fused_v.step(vel[0], uncond=None if unc is None else unc[0], g=request.guidance_scale)
                    if with_sound:
                        fused_s.step(vel[1], uncond=None if unc is None else unc[1], g=request.guidance_scale)
                    continue
                vel = self.guided(run, request.guidance_scale, do_cfg)
                video = uni_v.step(vel[0], timestep, video)
                if with_sound:
                    sound = uni_s.step(vel[1], timestep, sound)
                if cond_latents is not None:
                    video[:, :, cond_idx] = cond_latents[:, :, cond_idx]
        self._close_slot(slot)
        if slot.tensors:
            video = video.clone()              # the slot's tensor is overwritten by the next request
        if with_sound:
            return {"video": video, "sound": sound.transpose(1, 2).contiguous()}
        return video

    # ---- decode helpers (need the optional VAE / AVAE)
    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        if self.vae is None:
            raise RuntimeError("scheduler built without a VAE")
        from .vae_wan import decode_auto

        return ((decode_auto(self.vae, latents.to(self.dtype)).float() + 1.0) / 2.0).clamp(0.0, 1.0)

    @torch.no_grad()
    def encode(self, pixels: torch.Tensor) -> torch.Tensor:
        if self.vae is None:
            raise RuntimeError("scheduler built without a VAE")
        return self.vae.encode(pixels.to(self.device, self.dtype))

    @torch.no_grad()
    def decode_sound(self, sound_latent: torch.Tensor) -> torch.Tensor:
        if self.avae is None:
            raise RuntimeError("scheduler built without an AVAE")
        return self.avae.decode(sound_latent.to(self.device, self.dtype))

    @property
    def sound_sample_rate(self) -> int:
        if self.avae is None:
            raise RuntimeError("scheduler built without an AVAE")
        return self.avae.config.sample_rate


class Cosmos3PolicyScheduler(_GuidanceMixin, Scheduler):
    def __init__(self, transformer: Cosmos3Transformer, *, vae=None, device=None, flow_shift: float = 1.0,
                 use_karras_sigmas: bool = True) -> None:
        if not transformer.config.action_gen:
            raise ValueError("the policy scheduler needs a transformer built with action_gen=True")
        self.transformer = transformer
        self.device = torch.device(device) if device is not None else next(transformer.parameters()).device
        self.dtype = transformer.params_dtype
        self.latent_channel = transformer.config.latent_channel
        self.runner = Cosmos3Runner(transformer)
        self.vae = vae
        self._flow_shift, self._karras = flow_shift, use_karras_sigmas
        self._ready = False
        self._init_guidance()

    def setup(self) -> None:
        self._ready = True

    @torch.no_grad()
    def step(self, request: Cosmos3ActionRequest, *, decode_video: bool = False) -> dict[str, torch.Tensor]:
        if not self._ready:
            raise RuntimeError("call setup() before step()")
        if request.mode not in ACTION_MODES:
            raise ValueError(f"mode must be one of {ACTION_MODES}, got {request.mode!r}")
        if request.cond_video_latents is None and request.cond_video_pixels is not None:
            if self.vae is None:
                raise RuntimeError("cond_video_pixels given but the scheduler has no VAE to encode them")
            request = dataclasses.replace(request, cond_video_latents=self.vae.encode(
                request.cond_video_pixels.to(self.device, self.dtype)))
        dev, dt = self.device, self.dtype
        t_lat, h_lat, w_lat = request.video_shape
        chunk, ad, raw = request.action_chunk, request.action_dim, request.raw_action_dim
        B = request.text_ids.shape[0]
        domain = torch.full((B,), request.domain_id, device=dev, dtype=torch.long)
        if request.cond_frame_indexes is not None:
            clean = list(request.cond_frame_indexes)
        else:
            clean = list(range(t_lat)) if request.mode == "inverse_dynamics" else [0]
        action_clean = request.mode == "forward_dynamics"
        video = seeded_normal((B, self.latent_channel, t_lat, h_lat, w_lat), request.seed, dev, dt)
        action = seeded_normal((B, chunk, ad), request.seed, dev, dt)
        action[:, :, raw:] = 0.0
        cond_video = request.cond_video_latents.to(dev, dt) if request.cond_video_latents is not None else None
        if cond_video is not None:
            video[:, :, clean] = cond_video[:, :, clean]
        cond_action = request.cond_action.to(dev, dt) if request.cond_action is not None else None
        if action_clean and cond_action is not None:
            action = cond_action.clone()
            action[:, :, raw:] = 0.0
        vmask = torch.ones(B, t_lat, dtype=torch.bool, device=dev)
        vmask[:, clean] = False
        amask = torch.full((B, chunk), not action_clean, dtype=torch.bool, device=dev)
        prompts = {"cond": (request.text_ids.to(dev), request.text_mask.to(dev)),
                   "uncond": (request.neg_text_ids.to(dev), request.neg_text_mask.to(dev))}
        do_cfg = request.guidance_scale > 1.0
        mk = lambda: UniPCMultistepSampler(flow_shift=self._flow_shift, use_karras_sigmas=self._karras)  # noqa: E731
        uni_v, uni_a = mk(), mk()
        uni_v.set_timesteps(request.num_inference_steps, device=dev)
        uni_a.set_timesteps(request.num_inference_steps, device=dev)
        fused = self.fused_sampler and FusedUniPCStream.usable(video)
        branches = ("cond", "uncond") if do_cfg else ("cond",)
        slot = self._loop_slot(("action", tuple(video.shape), tuple(action.shape),
                                tuple(real_text_len(prompts[b][1]) for b in branches)), fused)
        self.runner.reset(slot.conds if slot.persistent else None)
        if slot.persistent:
            # a captured step reads the slot's tensors and conditions: this request's values go into them
            video, action, domain = slot.hold("video", video), slot.hold("action", action), slot.hold("domain", domain)
            vmask, amask = slot.hold("vmask", vmask), slot.hold("amask", amask)
            for b in branches:
                self.runner.prepare(b, text_ids=prompts[b][0], text_mask=prompts[b][1], video_shape=request.video_shape,
                                    fps=request.fps, action_len=chunk)
        fused_v = fused_a = None
        if fused:
            video, action = video.contiguous(), action.contiguous()
            fused_v = FusedUniPCStream(uni_v, video, view=(video.shape[1], t_lat, h_lat * w_lat),
                                       keep=None if cond_video is None else ~vmask, cond=cond_video)
            held = action_clean and cond_action is not None     # forward dynamics: the action stream stays the given one
            fused_a = FusedUniPCStream(uni_a, action, view=(1, chunk, ad), live_inner=raw,
                                       keep=torch.ones(B, chunk, dtype=torch.bool, device=dev) if held else None,
                                       cond=action.clone() if held else None)
        graph = slot.graph
        tval = slot.hold("tval", torch.empty(1, device=dev, dtype=dt))      # one buffer for all steps: a captured step reads it
        with event_scope("cosmos3.policy_denoise_loop"):
            for timestep in uni_v.timesteps:
                tval.copy_(timestep.reshape(1))

                def run(branch: str):
                    ids, mask = prompts[branch]
                    return self.runner.forward(branch, video, tval, text_ids=ids, text_mask=mask,
                                               video_shape=request.video_shape, fps=request.fps, noisy_frame_mask=vmask,
                                               action_latents=action, action_domain_id=domain, action_noisy_mask=amask)

                if fused_v is not None:
                    vel, unc = graph.run(lambda: self.guided_pair(run, request.guidance_scale, do_cfg))
                    fused_v.step(vel[0], uncond=None if unc is None else unc[0], g=request.guidance_scale)
                    fused_a.step(vel[1], uncond=None if unc is None else unc[1], g=request.guidance_scale)
                    continue
                v_vel, a_vel = self.guided(run, request.guidance_scale, do_cfg)
                a_vel = a_vel.clone()
                a_vel[:, :, raw:] = 0.0
                video = uni_v.step(v_vel, timestep, video)
                action = uni_a.step(a_vel, timestep, action)
                if cond_video is not None:
                    video[:, :, clean] = cond_video[:, :, clean]
                if action_clean and cond_action is not None:
                    action = cond_action.to(action.dtype).clone()
                    action[:, :, raw:] = 0.0
        self._close_slot(slot)
        if slot.tensors:
            video, action = video.clone(), action.clone()      # the slot's tensors are overwritten by the next request
        out = {"video": video, "action": action[:, :, :raw]}
        if decode_video:
            if self.vae is None:
                raise RuntimeError("decode_video=True but the scheduler was built without a VAE")
            from .vae_wan import decode_auto

            out["pixels"] = ((decode_auto(self.vae, video).float() + 1.0) / 2.0).clamp(0.0, 1.0)
        return out


# the multi-GPU plugin names share the implementation: parallelism comes from the mesh
Cosmos3T2VWNScheduler = Cosmos3T2VScheduler
Cosmos3PolicyWNScheduler = Cosmos3PolicyScheduler

__all__ = ["Cosmos3T2VRequest", "Cosmos3ActionRequest", "ACTION_MODES", "pixel_to_latent_shape", "seeded_normal",
           "Cosmos3Runner", "StepGraph", "LoopSlot", "Cosmos3T2VScheduler", "Cosmos3PolicyScheduler", "Cosmos3T2VWNScheduler",
           "Cosmos3PolicyWNScheduler"]
