"""Pre/post-processing pipelines around the serving engines.

A pipeline is a list of registered steps that pass one mutable dict (the *transition*) along.
Pipelines read and write the lerobot checkpoint layout: ``policy_preprocessor.json`` /
``policy_postprocessor.json`` with ``{name, steps: [{registry_name, config, state_file?}]}`` and
normaliser statistics in safetensors sidecars keyed ``"<feature>.<stat>"``, so the processors that
ship with public Pi0 / Pi0.5 checkpoints load unchanged.

Reference: phyai-utils-tools/src/phyai_utils_tools/processing/{types,transition,pipeline,base_processor}.py,
processing/ops/image_ops.py, processing/steps/*.py.
"""

from __future__ import annotations

import abc
import json
import re
from dataclasses import dataclass, field
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Iterable, Sequence

import torch
import torch.nn.functional as F

# ---------------------------------------------------------------- types (values match lerobot's enums)
class FeatureType(str, Enum):
    STATE = "STATE"
    VISUAL = "VISUAL"
    ENV = "ENV"
    ACTION = "ACTION"
    REWARD = "REWARD"
    LANGUAGE = "LANGUAGE"


class NormalizationMode(str, Enum):
    MIN_MAX = "MIN_MAX"
    MEAN_STD = "MEAN_STD"
    IDENTITY = "IDENTITY"
    QUANTILES = "QUANTILES"
    QUANTILE10 = "QUANTILE10"


@dataclass(frozen=True)
class PolicyFeature:
    type: FeatureType
    shape: tuple[int, ...]


# ---------------------------------------------------------------- transition keys
IMAGES, STATE, TASK = "images", "state", "task"
PROMPT, PIXEL_VALUES, INPUT_IDS, LANG_LENS = "prompt", "pixel_values", "input_ids", "lang_lens"
ACTION = "action"
Transition = dict


def identity_adapter(x: Any) -> Any:
    return x


# ---------------------------------------------------------------- registry / step / pipeline
class ProcessorStepError(Exception):
    pass


class ProcessorStepRegistry:
    _registry: dict[str, type] = {}

    @classmethod
    def register(cls, name: str | None = None) -> Callable[[type], type]:
        def deco(step_cls: type) -> type:
            key = name or step_cls.__name__
            if key in cls._registry and cls._registry[key] is not step_cls:
                raise ValueError(f"processor step {key!r} is already registered")
            cls._registry[key] = step_cls
            step_cls._registry_name = key
            return step_cls
        return deco

    @classmethod
    def get(cls, name: str) -> type:
        if name not in cls._registry:
            raise KeyError(f"unknown processor step {name!r}; registered: {sorted(cls._registry)}")
        return cls._registry[name]

    @classmethod
    def list(cls) -> list[str]:
        return sorted(cls._registry)

    @classmethod
    def unregister(cls, name: str) -> None:
        cls._registry.pop(name, None)


class ProcessorStep(abc.ABC):
    """One transform of the transition. Serialisable through ``get_config`` (json) and ``state_dict`` (tensors)."""

    @abc.abstractmethod
    def __call__(self, transition: Transition) -> Transition: ...

    def get_config(self) -> dict[str, Any]:
        return {}

    def state_dict(self) -> dict[str, torch.Tensor]:
        return {}

    def load_state_dict(self, state: dict[str, torch.Tensor]) -> None:
        return None

    def reset(self) -> None:
        return None


@dataclass
class ProcessorPipeline:
    steps: Sequence[ProcessorStep] = field(default_factory=list)
    name: str = "ProcessorPipeline"
    to_transition: Callable[[Any], Transition] = field(default=identity_adapter, repr=False)
    to_output: Callable[[Transition], Any] = field(default=identity_adapter, repr=False)

    def __call__(self, data: Any) -> Any:
        t = self.to_transition(data)
        for s in self.steps:
            t = s(t)
        return self.to_output(t)

    def step_through(self, data: Any) -> Iterable[Transition]:
        t = self.to_transition(data)
        yield dict(t)
        for s in self.steps:
            t = s(t)
            yield dict(t)

    def reset(self) -> None:
        for s in self.steps:
            s.reset()

    def __len__(self) -> int:
        return len(self.steps)

    def __getitem__(self, i: int) -> ProcessorStep:
        return self.steps[i]

    def get_config(self) -> dict[str, Any]:
        return {"name": self.name, "steps": [{"registry_name": getattr(type(s), "_registry_name", type(s).__name__),
                                               "config": s.get_config()} for s in self.steps]}

    # ---- persistence
    def save_pretrained(self, save_directory: str | Path, *, config_filename: str | None = None) -> Path:
        from safetensors.torch import save_file

        d = Path(save_directory)
        d.mkdir(parents=True, exist_ok=True)
        stem = re.sub(r"[^a-zA-Z0-9_]", "_", self.name.lower())
        cfg: dict[str, Any] = {"name": self.name, "steps": []}
        for i, s in enumerate(self.steps):
            rn = getattr(type(s), "_registry_name", type(s).__name__)
            entry: dict[str, Any] = {"registry_name": rn, "config": s.get_config()}
            state = s.state_dict()
            if state:
                fname = f"{stem}_step_{i}_{rn}.safetensors"
                save_file({k: v.detach().cpu().contiguous() for k, v in state.items()}, str(d / fname))
                entry["state_file"] = fname
            cfg["steps"].append(entry)
        out = d / (config_filename or f"{stem}.json")
        out.write_text(json.dumps(cfg, indent=2))
        return out

    @classmethod
    def from_pretrained(cls, src: str | Path, config_filename: str, *, name: str | None = None,
                        overrides: dict[str, dict[str, Any]] | None = None, step_kwargs: dict[str, dict[str, Any]] | None = None,
                        to_transition=None, to_output=None) -> "ProcessorPipeline":
        """``overrides[registry_name]`` replace saved config values; ``step_kwargs[registry_name]`` inject objects a json
        cannot carry (a tokenizer, a device). An unknown step name is an error, never skipped."""
        path = Path(src)
        if path.is_dir():
            cfg_path, base = path / config_filename, path
        elif path.is_file():
            cfg_path, base = path, path.parent
        else:
            raise FileNotFoundError(f"{src} is neither a directory nor a file (hub download is not available offline)")
        if not cfg_path.is_file():
            raise FileNotFoundError(f"{config_filename} not found in {base}")
        cfg = json.loads(cfg_path.read_text())
        overrides, step_kwargs = overrides or {}, step_kwargs or {}
        steps = []
        for entry in cfg.get("steps", []):
            rn = entry.get("registry_name")
            if rn is None:
                raise ProcessorStepError(f"step entry without 'registry_name': {entry!r}")
            try:
                step_cls = ProcessorStepRegistry.get(rn)
            except KeyError as e:
                raise ProcessorStepError(f"unknown processor step {rn!r}; implemented: {ProcessorStepRegistry.list()}") from e
            merged = {**entry.get("config", {}), **overrides.get(rn, {}), **step_kwargs.get(rn, {})}
            try:
                step = step_cls(**merged)
            except Exception as e:
                raise ProcessorStepError(f"cannot build step {rn!r} from {merged!r}: {e}") from e
            if entry.get("state_file"):
                from safetensors.torch import load_file

                f = base / entry["state_file"]
                if not f.is_file():
                    raise FileNotFoundError(f"step {rn!r} names state file {entry['state_file']!r}, missing at {f}")
                step.load_state_dict(load_file(str(f)))
            steps.append(step)
        return cls(steps=steps, name=name or cfg.get("name", "ProcessorPipeline"),
                   to_transition=to_transition or identity_adapter, to_output=to_output or identity_adapter)


class BaseModelProcessor(abc.ABC):
    """A model's pair of pipelines: ``preprocess(raw) -> engine request fields`` and ``postprocess(output)``."""

    preprocessor: ProcessorPipeline
    postprocessor: ProcessorPipeline

    @abc.abstractmethod
    def build_preprocessor(self) -> ProcessorPipeline: ...

    @abc.abstractmethod
    def build_postprocessor(self) -> ProcessorPipeline: ...

    def preprocess(self, data: Any) -> Any:
        return self.preprocessor(data)

    def postprocess(self, data: Any) -> Any:
        return self.postprocessor(data)


# ---------------------------------------------------------------- image ops
def resize_with_pad(images: torch.Tensor, target_h: int, target_w: int, *, mode: str = "bilinear", pad_value: float = 0.0) -> torch.Tensor:
    """(B, C, H, W): shrink/grow without distortion to fit the target, then pad symmetrically."""
    if images.dim() != 4:
        raise ValueError(f"resize_with_pad expects (B, C, H, W), got {tuple(images.shape)}")
    _, _, h, w = images.shape
    if (h, w) == (target_h, target_w):
        return images
    if images.dtype != torch.uint8 and not images.dtype.is_floating_point:
        raise ValueError(f"unsupported image dtype {images.dtype}")
    ratio = max(w / target_w, h / target_h)
    rh, rw = int(h / ratio), int(w / ratio)
    kw = dict(size=(rh, rw), mode=mode, align_corners=False if mode == "bilinear" else None)
    if images.dtype == torch.uint8:
        # bytes are interpolated as bytes where the device has that kernel (the CPU does: same pixels as the reference,
        # phyai-utils-tools/src/phyai_utils_tools/processing/ops/image_ops.py:56-64), else through fp32
        try:
            out = F.interpolate(images, **kw)
        except (RuntimeError, NotImplementedError):
            out = F.interpolate(images.float(), **kw)
        out = out.round().clamp(0, 255).to(torch.uint8)
    else:
        out = F.interpolate(images, **kw)
    top, rem_h = divmod(target_h - rh, 2)
    left, rem_w = divmod(target_w - rw, 2)
    return F.pad(out, (left, left + rem_w, top, top + rem_h), value=pad_value)


def normalize_pixels(images: torch.Tensor) -> torch.Tensor:
    """[0, 1] -> [-1, 1]."""
    return images * 2.0 - 1.0


# ---------------------------------------------------------------- generic steps
@ProcessorStepRegistry.register("resize_with_pad_step")
@dataclass
class ResizeWithPadStep(ProcessorStep):
    """``images`` (list of per-camera (B, C, H, W) or stacked (B, n, C, H, W)) -> ``pixel_values`` (B, n, C, h, w).

    The target is ``height`` x ``width``, or ``target_size`` squared (the reference's spelling:
    phyai-utils-tools/src/phyai_utils_tools/processing/steps/image_steps.py:31-45). ``num_images`` / ``num_channels``, when
    given, are checked against what arrives (a wrong camera count or channel count is an error, not a silent reshape)."""

    height: int = 224
    width: int = 224
    pad_value: float = 0.0
    mode: str = "bilinear"
    target_size: int | None = None
    num_images: int | None = None
    num_channels: int | None = None

    def __post_init__(self) -> None:
        if self.target_size is not None:
            self.height = self.width = int(self.target_size)

    def __call__(self, t: Transition) -> Transition:
        imgs = t[IMAGES]
        if isinstance(imgs, torch.Tensor):
            if imgs.dim() != 5:
                raise ValueError(f"stacked images are (B, num_images, C, H, W), got {tuple(imgs.shape)}")
            cams = list(imgs.unbind(1))
        else:
            cams = list(imgs)
        if self.num_images is not None and len(cams) != self.num_images:
            raise ValueError(f"expected {self.num_images} cameras, got {len(cams)}")
        for i, c in enumerate(cams):
            if c.dim() != 4:
                raise ValueError(f"camera {i} is (B, C, H, W), got {tuple(c.shape)}")
            if self.num_channels is not None and c.shape[1] != self.num_channels:
                raise ValueError(f"camera {i} has {c.shape[1]} channels, expected {self.num_channels}")
        out = dict(t)
        out[PIXEL_VALUES] = torch.stack([resize_with_pad(c, self.height, self.width, mode=self.mode, pad_value=self.pad_value)
                                         for c in cams], dim=1)
        return out

    def get_config(self):
        cfg = {"height": self.height, "width": self.width, "pad_value": self.pad_value, "mode": self.mode}
        if self.num_images is not None:
            cfg["num_images"] = self.num_images
        if self.num_channels is not None:
            cfg["num_channels"] = self.num_channels
        return cfg


@ProcessorStepRegistry.register("normalize_image_step")
@dataclass
class NormalizeImageStep(ProcessorStep):
    def __call__(self, t: Transition) -> Transition:
        t[PIXEL_VALUES] = normalize_pixels(t[PIXEL_VALUES].float() / (255.0 if t[PIXEL_VALUES].dtype == torch.uint8 else 1.0))
        return t


_FIELD_OF = {FeatureType.STATE: STATE, FeatureType.ACTION: ACTION}


def _apply_norm(x, mode: NormalizationMode, s: dict, eps: float, inverse: bool):
    pairs = {NormalizationMode.MIN_MAX: ("min", "max"), NormalizationMode.QUANTILES: ("q01", "q99"),
             NormalizationMode.QUANTILE10: ("q10", "q90")}
    if mode == NormalizationMode.MEAN_STD:
        return x * (s["std"] + eps) + s["mean"] if inverse else (x - s["mean"]) / (s["std"] + eps)
    if mode in pairs:
        lo, hi = (s[k] for k in pairs[mode])
        return (x + 1.0) / 2.0 * (hi - lo + eps) + lo if inverse else (x - lo) / (hi - lo + eps) * 2.0 - 1.0
    return x


@dataclass
class _NormalizeBase(ProcessorStep):
    features: dict = field(default_factory=dict)
    norm_map: dict = field(default_factory=dict)
    stats: dict | None = None
    device: Any = None
    dtype: torch.dtype = torch.float32
    eps: float = 1e-8
    inverse = False

    def __post_init__(self) -> None:
        self._features = {n: f if isinstance(f, PolicyFeature) else PolicyFeature(FeatureType(f["type"]), tuple(f.get("shape", ())))
                          for n, f in (self.features or {}).items()}
        self._norm_map = {(k if isinstance(k, FeatureType) else FeatureType(k)): (v if isinstance(v, NormalizationMode) else NormalizationMode(v))
                          for k, v in (self.norm_map or {}).items()}
        self._explicit = bool(self.stats)
        self._stats = {n: {k: torch.as_tensor(v, dtype=self.dtype, device=self.device) for k, v in sub.items()}
                       for n, sub in (self.stats or {}).items()}

    def __call__(self, t: Transition) -> Transition:
        for name, feat in self._features.items():
            key = _FIELD_OF.get(feat.type)
            mode = self._norm_map.get(feat.type, NormalizationMode.IDENTITY)
            if key is None or key not in t or t[key] is None or name not in self._stats or mode == NormalizationMode.IDENTITY:
                continue
            x = t[key]
            s = {k: v.to(x.device) for k, v in self._stats[name].items()}
            width = next(iter(s.values())).shape[-1]
            if x.shape[-1] < width:
                raise ValueError(f"{name}: tensor width {x.shape[-1]} is smaller than the statistics' {width}")
            head = _apply_norm(x[..., :width].to(self.dtype), mode, s, self.eps, self.inverse)
            t[key] = torch.cat([head.to(x.dtype), x[..., width:]], dim=-1) if x.shape[-1] > width else head.to(x.dtype)
        return t

    def get_config(self):
        return {"eps": self.eps, "features": {n: {"type": f.type.value, "shape": list(f.shape)} for n, f in self._features.items()},
                "norm_map": {k.value: v.value for k, v in self._norm_map.items()}}

    def state_dict(self):
        return {f"{n}.{k}": v.detach().cpu() for n, sub in self._stats.items() for k, v in sub.items()}

    def load_state_dict(self, state) -> None:
        if self._explicit:          # statistics given at construction win over a sidecar
            return
        nested: dict[str, dict[str, torch.Tensor]] = {}
        for flat, v in state.items():
            n, _, k = flat.rpartition(".")
            nested.setdefault(n, {})[k] = v.to(dtype=self.dtype, device=self.device)
        self._stats = nested


@ProcessorStepRegistry.register("normalizer_processor")
@dataclass
class NormalizerStep(_NormalizeBase):
    inverse = False


@ProcessorStepRegistry.register("unnormalizer_processor")
@dataclass
class UnnormalizerStep(_NormalizeBase):
    inverse = True


@ProcessorStepRegistry.register("tokenizer_processor")
@dataclass
class TokenizerStep(ProcessorStep):
    """``prompt`` (else ``task``) -> ``input_ids`` (B, max_length) right-padded and ``lang_lens`` (B,). A prompt built by an
    earlier step always wins; ``task_key`` (``"task"`` in lerobot's json) names the raw text read when there is none."""

    tokenizer: Any = None
    tokenizer_name: str | None = None
    max_length: int = 200
    task_key: str = TASK
    padding_side: str = "right"
    padding: str = "max_length"
    truncation: bool = True

    def __post_init__(self) -> None:
        if self.tokenizer is None and self.tokenizer_name:
            from .tokenizer import get_tokenizer

            self.tokenizer = get_tokenizer(self.tokenizer_name)

    def __call__(self, t: Transition) -> Transition:
        if self.tokenizer is None:
            raise ProcessorStepError("tokenizer_processor needs a tokenizer (pass step_kwargs={'tokenizer_processor': {'tokenizer': tok}})")
        texts = t.get(PROMPT) or t.get(self.task_key) or t.get(TASK)
        if texts is None:
            raise ProcessorStepError("tokenizer_processor needs a 'prompt' or 'task' entry")
        if isinstance(texts, str):
            texts = [texts]
        enc = self.tokenizer(list(texts), max_length=self.max_length, padding=self.padding, truncation=self.truncation,
                             return_tensors="pt", padding_side=self.padding_side) if _accepts_side(self.tokenizer) else \
            self.tokenizer(list(texts), max_length=self.max_length, padding=self.padding, truncation=self.truncation, return_tensors="pt")
        t[INPUT_IDS] = enc["input_ids"].long()
        t[LANG_LENS] = enc["attention_mask"].sum(-1).long()
        return t

    def get_config(self):
        return {"max_length": self.max_length, "task_key": self.task_key, "padding_side": self.padding_side,
                "padding": self.padding, "truncation": self.truncation, "tokenizer_name": self.tokenizer_name}


def _accepts_side(tok) -> bool:
    return bool(getattr(tok, "accepts_padding_side", False))


@ProcessorStepRegistry.register("device_processor")
@dataclass
class DeviceStep(ProcessorStep):
    """Tensors (and lists of tensors) to ``device``; floating ones to ``float_dtype`` (a ``torch.dtype`` or its name)."""

    device: Any = "cpu"
    float_dtype: Any = None

    def __call__(self, t: Transition) -> Transition:
        dt = getattr(torch, self.float_dtype) if isinstance(self.float_dtype, str) else self.float_dtype
        for k, v in list(t.items()):
            if isinstance(v, torch.Tensor):
                v = v.to(self.device, non_blocking=True)
                t[k] = v.to(dt) if dt is not None and v.dtype.is_floating_point else v
            elif isinstance(v, (list, tuple)) and v and all(isinstance(e, torch.Tensor) for e in v):
                t[k] = type(v)(e.to(self.device, non_blocking=True) for e in v)
        return t

    def get_config(self):
        return {"device": str(self.device), "float_dtype": None if self.float_dtype is None else str(self.float_dtype).replace("torch.", "")}


@ProcessorStepRegistry.register("to_batch_processor")
@dataclass
class AddBatchDimensionStep(ProcessorStep):
    """Unbatched sample -> batch of one (state 1-D, images 3-D, task a single string)."""

    def __call__(self, t: Transition) -> Transition:
        if isinstance(t.get(STATE), torch.Tensor) and t[STATE].dim() == 1:
            t[STATE] = t[STATE][None]
        if isinstance(t.get(ACTION), torch.Tensor) and t[ACTION].dim() <= 2 and t.get("_unbatched_action", True) and t[ACTION].dim() == 1:
            t[ACTION] = t[ACTION][None]
        imgs = t.get(IMAGES)
        if isinstance(imgs, (list, tuple)):
            t[IMAGES] = [i[None] if i.dim() == 3 else i for i in imgs]
        elif isinstance(imgs, torch.Tensor) and imgs.dim() == 4:
            t[IMAGES] = imgs[None]
        if isinstance(t.get(TASK), str):
            t[TASK] = [t[TASK]]
        return t


@ProcessorStepRegistry.register("rename_observations_processor")
@dataclass
class RenameObservationsStep(ProcessorStep):
    rename_map: dict = field(default_factory=dict)

    def __call__(self, t: Transition) -> Transition:
        for old, new in self.rename_map.items():
            if old in t:
                t[new] = t.pop(old)
        return t

    def get_config(self):
        return {"rename_map": dict(self.rename_map)}


@ProcessorStepRegistry.register("slice_action_step")
@dataclass
class SliceActionStep(ProcessorStep):
    """Keep the first ``action_dim`` channels (models pad actions to a fixed width)."""

    action_dim: int | None = None

    def __call__(self, t: Transition) -> Transition:
        if self.action_dim is not None and t.get(ACTION) is not None:
            t[ACTION] = t[ACTION][..., :self.action_dim]
        return t

    def get_config(self):
        return {"action_dim": self.action_dim}


__all__ = ["FeatureType", "NormalizationMode", "PolicyFeature", "IMAGES", "STATE", "TASK", "PROMPT", "PIXEL_VALUES", "INPUT_IDS",
           "LANG_LENS", "ACTION", "Transition", "identity_adapter", "ProcessorStepError", "ProcessorStepRegistry", "ProcessorStep",
           "ProcessorPipeline", "BaseModelProcessor", "resize_with_pad", "normalize_pixels", "ResizeWithPadStep", "NormalizeImageStep",
           "NormalizerStep", "UnnormalizerStep", "TokenizerStep", "DeviceStep", "AddBatchDimensionStep", "RenameObservationsStep",
           "SliceActionStep"]
