"""Plugins ``cosmos3`` / ``cosmos3_wn``: text/image-to-video [+ sound] generation.

A checkpoint directory holds ``transformer/``, ``vae/``, ``sound_tokenizer/`` and
``scheduler/``. Without one (``checkpoint_dir=None`` and an explicit ``config``) the networks are
built with seeded random weights, which is what shape tests and synthetic benchmarks use.

Reference: phyai/src/phyai/models/cosmos3/main_cosmos3.py:41-201, main_cosmos3_wn.py:53-189.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from pathlib import Path
from typing import ClassVar

import torch

from ...engine import Engine, Entry, EntryArgs
from ...engine_config import get_engine_config
from ...layers.quant import load_quant_plan, use_quant_plan
from ...utils.checkpoint import load_config
from ...utils.logging import this_rank_log
from ...weights import load_pretrained
from .avae_sound import Cosmos3AVAESoundDecoder, cosmos3_avae_weight_remap
from .configuration_cosmos3 import Cosmos3AVAESoundConfig, Cosmos3Config, Cosmos3WanVAEConfig
from .sampler_unipc import resolve_use_karras_sigmas
from .scheduler_cosmos3 import Cosmos3T2VRequest, Cosmos3T2VScheduler
from .transformer_cosmos3 import Cosmos3Transformer, cosmos3_weight_remap
from .vae_wan import Cosmos3WanVAE, cosmos3_vae_weight_remap

logger = logging.getLogger(__name__)


@dataclass
class Cosmos3Args(EntryArgs):
    checkpoint_dir: str | Path | None = None
    config: Cosmos3Config | None = None
    flow_shift: float = 10.0
    use_karras_sigmas: bool | None = False   # False: linear flow schedule with flow_shift; None: read the checkpoint
    load_sound: bool | None = None           # None: follow config.sound_gen
    load_vae: bool = True
    vae_config: Cosmos3WanVAEConfig | None = None
    avae_config: Cosmos3AVAESoundConfig | None = None
    weight_strict: bool = False
    random_init_seed: int = 0
    # accepted so that argument bundles written for the reference load: nothing here goes through torch.compile (the GEN
    # tower runs this package's kernels, on one GPU as a CUDA graph per request geometry), so the two are not acted on
    torch_compile: bool = False
    compile_kwargs: dict | None = None


def wants_sound(args, config: Cosmos3Config) -> bool:
    return bool(config.sound_gen) if args.load_sound is None else bool(args.load_sound)


def build_transformer(args, ckpt: Path | None, device, dtype) -> Cosmos3Transformer:
    if args.config is not None:
        config = args.config
    elif ckpt is not None:
        config = load_config(ckpt / "transformer", Cosmos3Config)
    else:
        raise ValueError("give checkpoint_dir, or config for a randomly initialised network")
    with use_quant_plan(load_quant_plan(ckpt / "transformer" if ckpt is not None else None)):
        tr = Cosmos3Transformer(config, params_dtype=dtype, device=device).eval()
    if ckpt is not None:
        load_pretrained(tr, ckpt / "transformer", remap=cosmos3_weight_remap, strict=args.weight_strict)
    else:
        tr.init_random(args.random_init_seed)
    return tr


def _seeded_fill(module: torch.nn.Module, seed: int) -> None:
    g = torch.Generator().manual_seed(seed)
    for p in module.parameters():
        if p.dim() > 1 and p.shape[1:].numel() > 1:
            fan = p.shape[1:].numel()
            p.data.copy_((torch.randn(p.shape, generator=g) / fan ** 0.5).to(p.dtype))


def build_vae(args, ckpt: Path | None, device, dtype) -> Cosmos3WanVAE:
    cfg = args.vae_config if getattr(args, "vae_config", None) is not None else (
        load_config(ckpt / "vae", Cosmos3WanVAEConfig) if ckpt is not None else Cosmos3WanVAEConfig())
    vae = Cosmos3WanVAE(cfg, device=device, dtype=dtype).eval()
    if ckpt is not None:
        load_pretrained(vae, ckpt / "vae", remap=cosmos3_vae_weight_remap, strict=args.weight_strict)
    else:
        _seeded_fill(vae, args.random_init_seed + 1)
    return vae.to(device)


def build_avae(args, ckpt: Path | None, device, dtype) -> Cosmos3AVAESoundDecoder:
    cfg = args.avae_config if getattr(args, "avae_config", None) is not None else (
        load_config(ckpt / "sound_tokenizer", Cosmos3AVAESoundConfig) if ckpt is not None else Cosmos3AVAESoundConfig())
    avae = Cosmos3AVAESoundDecoder(cfg, dtype=dtype, device=device).eval()
    if ckpt is not None:
        load_pretrained(avae, ckpt / "sound_tokenizer", remap=cosmos3_avae_weight_remap, strict=args.weight_strict)
    else:
        _seeded_fill(avae, args.random_init_seed + 2)
    return avae


@Engine.register
class Cosmos3Entry(Entry):
    name: ClassVar[str] = "cosmos3"
    args_cls: ClassVar[type[EntryArgs]] = Cosmos3Args

    def __init__(self) -> None:
        self.transformer: Cosmos3Transformer | None = None
        self.vae: Cosmos3WanVAE | None = None
        self.avae: Cosmos3AVAESoundDecoder | None = None
        self.scheduler: Cosmos3T2VScheduler | None = None

    def setup(self, args: Cosmos3Args) -> None:  # type: ignore[override]
        eng = get_engine_config()
        device, dtype = eng.device.target, eng.device.params_dtype
        ckpt = Path(args.checkpoint_dir) if args.checkpoint_dir is not None else None
        self.transformer = build_transformer(args, ckpt, device, dtype)
        if args.load_vae:
            self.vae = build_vae(args, ckpt, device, dtype)
        if wants_sound(args, self.transformer.config):
            self.avae = build_avae(args, ckpt, device, dtype)
        karras = resolve_use_karras_sigmas(args.use_karras_sigmas, ckpt)
        self.scheduler = Cosmos3T2VScheduler(self.transformer, vae=self.vae, avae=self.avae, device=device,
                                             flow_shift=args.flow_shift, use_karras_sigmas=karras)
        self.scheduler.setup()
        this_rank_log(logger, logging.INFO, "%s ready (cfg=%d, sound=%s, flow_shift=%s, karras=%s)", self.name,
                      self.scheduler.cfg_size, self.avae is not None, args.flow_shift, karras)

    def step(self, request: Cosmos3T2VRequest, *, decode: bool = True):  # type: ignore[override]
        """Pixels (B, 3, T, H, W) in [0, 1]; with sound a dict ``video / sound / sample_rate``.
        ``decode=False`` (or a plugin built without a VAE) returns the latents."""
        if self.scheduler is None:
            raise RuntimeError(f"{type(self).__name__}.step before setup")
        out = self.scheduler.step(request)
        if not decode or self.vae is None:
            return out
        if isinstance(out, dict):
            return {"video": self.scheduler.decode(out["video"]), "sound": self.scheduler.decode_sound(out["sound"]),
                    "sample_rate": self.scheduler.sound_sample_rate}
        return self.scheduler.decode(out)

    def close(self) -> None:
        if self.scheduler is not None:
            self.scheduler.close()
        self.scheduler = self.transformer = self.vae = self.avae = None

    def dump_targets(self):
        return {} if self.transformer is None else {"transformer": self.transformer}


__all__ = ["Cosmos3Args", "Cosmos3Entry", "build_transformer", "build_vae", "build_avae", "wants_sound"]
