"""Cosmos3 prompt, image and action processing for the generation and policy plugins.

* ``Cosmos3Processor``: chat-template tokenisation of the positive / negative prompt, with the
  duration / resolution metadata the model was trained to see appended to the positive one.
* ``Cosmos3GenerationPostProcessor``: pixels in [0, 1] -> uint8 frames (+ writers).
* ``Cosmos3PolicyProcessor``: observation frame(s) -> pixels at the training bucket (bicubic shrink, reflected
  margins), plain or structured JSON caption -> ids, conditioning actions padded to the model width, embodiment
  name -> domain id; predicted actions back to the robot's units.

Reference: phyai-utils-tools/src/phyai_utils_tools/models/cosmos3/{steps_cosmos3,processor_cosmos3}.py.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np
import torch

from .processing import (IMAGES, PIXEL_VALUES, TASK, BaseModelProcessor, ProcessorPipeline, ProcessorStep, ProcessorStepRegistry,
                         Transition)

TEXT_IDS, TEXT_MASK, NEG_TEXT_IDS, NEG_TEXT_MASK = "text_ids", "text_mask", "neg_text_ids", "neg_text_mask"
COND_ACTION, DOMAIN_ID, MODE, ACTION_CHUNK, RAW_ACTION_DIM, VIDEO_SHAPE = "cond_action", "domain_id", "mode", "action_chunk", "raw_action_dim", "video_shape"
META_HEIGHT, META_WIDTH = "meta_height", "meta_width"
COSMOS3_VISION_START_TOKEN = "<|vision_start|>"

# embodiment name -> id of its action adapter inside the checkpoint / width of its raw action vector
EMBODIMENT_TO_DOMAIN_ID = {"no_action": 0, "av": 1, "camera_pose": 2, "hand_pose": 3, "pusht": 4, "libero": 5, "umi": 6,
                           "bridge_orig_lerobot": 7, "droid_lerobot": 8, "robomind-franka": 8, "galbot": 9, "robomind-franka-dual": 12,
                           "robomind-ur": 13, "agibotworld": 15, "agibot_gear_gripper": 15, "agibot_gear_gripper_ext": 15, "fractal": 20}
EMBODIMENT_TO_RAW_ACTION_DIM = {"av": 9, "camera_pose": 9, "pusht": 2, "umi": 10, "bridge_orig_lerobot": 10, "droid_lerobot": 10,
                                "robomind-franka": 10, "robomind-franka-dual": 20, "robomind-ur": 10, "agibotworld": 29, "fractal": 10}
# training resolution buckets: tier -> aspect "w,h" -> (width, height); per tier the sides of the 1:1, 4:3 and 16:9 buckets
# (portrait buckets are the landscape ones transposed)
_TIER_SIDES = {"256": (256, (320, 256), (320, 192)), "480": (640, (736, 544), (832, 480)), "704": (960, (1088, 832), (1280, 704)),
               "720": (960, (1104, 832), (1280, 720)), "768": (1024, (1184, 880), (1360, 768)), "1080": (1440, (1664, 1248), (1920, 1080)),
               "1280": (1712, (1968, 1472), (2272, 1280)), "2048": (2728, (3160, 2368), (3640, 2048)),
               "gt_2048": (5464, (6304, 4728), (7280, 4096))}
VIDEO_RES_SIZE_INFO = {tier: {"1,1": (sq, sq), "4,3": four3, "3,4": four3[::-1], "16,9": wide, "9,16": wide[::-1]}
                       for tier, (sq, four3, wide) in _TIER_SIDES.items()}
# camera placement -> the sentence the action captions were written with
DEFAULT_VIEWPOINT_TEMPLATES = {
    "ego_view": "This video is captured from a first-person perspective looking at the scene.",
    "third_person_view": "This video is captured from a third-person perspective looking towards the agent from the front.",
    "wrist_view": "This video is captured from a wrist-mounted camera.",
    "concat_view": "This video contains concatenated views from multiple camera perspectives.",
}


def resolve_domain_id(domain: str | int) -> int:
    if isinstance(domain, int):
        if domain < 0:
            raise ValueError(f"domain_id must be non-negative, got {domain}")
        return domain
    key = str(domain).strip().lower()
    if key not in EMBODIMENT_TO_DOMAIN_ID:
        raise ValueError(f"unknown embodiment {domain!r}; known: {sorted(EMBODIMENT_TO_DOMAIN_ID)} (or pass an int)")
    return EMBODIMENT_TO_DOMAIN_ID[key]


def resolve_raw_action_dim(domain: str | int) -> int:
    if isinstance(domain, int):
        raise ValueError("an integer domain id does not say how wide its actions are: pass raw_action_dim")
    key = str(domain).strip().lower()
    if key not in EMBODIMENT_TO_RAW_ACTION_DIM:
        raise ValueError(f"no action width on record for {domain!r}: pass raw_action_dim")
    return EMBODIMENT_TO_RAW_ACTION_DIM[key]


def get_vision_data_resolution(spatial_shape: tuple[int, int]) -> str:
    """Tier of a frame of ``(height, width)``: the five 768-tier shapes by exact match, else by the shorter side."""
    h, w = int(spatial_shape[0]), int(spatial_shape[1])
    if (w, h) in VIDEO_RES_SIZE_INFO["768"].values():
        return "768"
    short = min(h, w)
    for limit, tier in ((256, "256"), (640, "480"), (960, "720")):
        if short <= limit:
            return tier
    raise ValueError(f"no resolution tier for a {h} x {w} frame")


def find_closest_target_size(h: int, w: int, resolution: str | int) -> tuple[int, int]:
    """``(width, height)`` of the bucket of this tier whose height / width ratio is nearest to ``h / w`` (the first of
    equally near buckets, in the order 1:1, 4:3, 3:4, 16:9, 9:16), as the reference picks it
    (phyai-utils-tools/src/phyai_utils_tools/models/cosmos3/steps_cosmos3.py:202-222)."""
    tier = VIDEO_RES_SIZE_INFO.get(str(resolution))
    if tier is None:
        raise ValueError(f"unknown resolution tier {resolution!r}; known: {list(VIDEO_RES_SIZE_INFO)}")
    ratio = h / w
    return min(tier.values(), key=lambda wh: abs(ratio - wh[1] / wh[0]))


def resolve_target_size(native_h: int, native_w: int, image_size: int) -> tuple[int, int]:
    """``(height, width)`` an observation frame is brought to: scale it to ``image_size`` rows, take the tier of that
    size and in it the bucket nearest in aspect ratio."""
    scaled_w = max(1, int(round(native_w * image_size / native_h)))
    tw, th = find_closest_target_size(image_size, scaled_w, get_vision_data_resolution((image_size, scaled_w)))
    return th, tw


def aspect_ratio_str(width: int, height: int) -> str:
    for tier in VIDEO_RES_SIZE_INFO.values():
        for ar, (w, h) in tier.items():
            if (w, h) == (width, height):
                return ar
    g = math.gcd(width, height)
    if g == 0:
        raise ValueError("width and height must be non-zero")
    return f"{width // g},{height // g}"


def cosmos3_action_json_caption(prompt: str, *, view_point: str, num_frames: int, fps: float, height: int, width: int) -> str:
    """Structured caption of an action rollout (what the policy variants are prompted with)."""
    dur = num_frames / float(fps)
    ok = dur >= 0 and math.isfinite(dur)
    minutes, seconds = divmod(round(dur) if ok else 0, 60)
    desc = prompt.strip()
    if not desc.endswith((".", "!", "?")):
        desc += "."
    out: dict[str, Any] = {}
    if DEFAULT_VIEWPOINT_TEMPLATES.get(view_point):
        out["cinematography"] = {"framing": DEFAULT_VIEWPOINT_TEMPLATES[view_point]}
    out["actions"] = [{"time": f"0:00-{minutes}:{seconds:02d}", "description": desc}]
    out["duration"] = f"{int(dur) if ok else 0}s"
    out["fps"] = float(fps)
    out["resolution"] = {"H": int(height), "W": int(width)}
    out["aspect_ratio"] = aspect_ratio_str(int(width), int(height))
    return json.dumps(out)


def cosmos3_generation_caption(prompt: str, *, fps: float, num_frames: int, height: int, width: int, aspect_ratio: str | None = None) -> str:
    """Positive prompt + duration / resolution metadata (JSON prompts get fields, plain text gets sentences)."""
    try:
        obj = json.loads(prompt)
    except (TypeError, ValueError):
        obj = None
    if isinstance(obj, dict):
        if num_frames > 1:
            obj["duration"], obj["fps"] = f"{int(num_frames / fps) if fps > 0 else 0}s", float(fps)
        else:
            obj.pop("duration", None)
            obj.pop("fps", None)
        obj["resolution"] = {"H": int(height), "W": int(width)}
        if aspect_ratio is not None:
            obj["aspect_ratio"] = aspect_ratio
        return json.dumps(obj)
    text = prompt.strip()
    if num_frames > 1:
        text = text.rstrip(".") + f". The video is {num_frames / float(fps):.1f} seconds long and is of {fps:.0f} FPS."
    return text.strip().rstrip(".") + f". This video is of {height}x{width} resolution."


def cosmos3_default_negative_prompt(path: str | Path | None = None) -> str:
    """The negative prompt used when the caller gives none. ``path``: a JSON file, re-serialised compactly the way the
    upstream sampler reads its ``negative_prompt_file`` (the model release ships one, ``neg_prompts.json``); without a
    file a short structured description of what a bad clip looks like."""
    if path is not None:
        return json.dumps(json.loads(Path(path).read_text()))
    return json.dumps({"quality": "low", "artifacts": ["blur", "flicker", "compression blocks", "banding", "noise"],
                       "motion": "jittery, frozen or physically implausible", "composition": "cropped subjects, distorted geometry",
                       "content": "text overlays, watermarks, duplicated limbs"})


@dataclass
class Cosmos3TokenizedPrompt:
    text_ids: torch.Tensor
    text_mask: torch.Tensor


def _flat_ids(out) -> list[int]:
    if isinstance(out, dict) or hasattr(out, "input_ids"):
        out = out["input_ids"]
    if hasattr(out, "tolist"):
        out = out.tolist()
    while out and isinstance(out[0], (list, tuple)):
        out = out[0]
    return [int(i) for i in out]


class Cosmos3Processor:
    def __init__(self, tokenizer_name_or_path: str | None = None, *, tokenizer: Any = None, use_system_prompt: bool = False,
                 fps: float | None = None, num_frames: int | None = None, height: int | None = None, width: int | None = None,
                 aspect_ratio: str | None = None, append_metadata: bool = True, negative_prompt: str | None = None,
                 negative_prompt_file: str | Path | None = None) -> None:
        if negative_prompt is None and negative_prompt_file is not None:
            negative_prompt = cosmos3_default_negative_prompt(negative_prompt_file)
        if tokenizer is None:
            from .tokenizer import get_tokenizer

            tokenizer = get_tokenizer(tokenizer_name_or_path)
        self.tokenizer, self.use_system_prompt = tokenizer, use_system_prompt
        self.fps, self.num_frames, self.height, self.width, self.aspect_ratio = fps, num_frames, height, width, aspect_ratio
        self.append_metadata, self._negative = bool(append_metadata), negative_prompt
        self.eos_token_id = int(tokenizer.eos_token_id)
        self.vision_start_token_id = int(tokenizer.convert_tokens_to_ids(COSMOS3_VISION_START_TOKEN))

    def _augment(self, prompt: str) -> str:
        if not self.append_metadata or None in (self.fps, self.num_frames, self.height, self.width):
            return prompt
        return cosmos3_generation_caption(prompt, fps=self.fps, num_frames=self.num_frames, height=self.height, width=self.width,
                                          aspect_ratio=self.aspect_ratio)

    def tokenize(self, prompt: str, *, device="cpu", augment: bool = True) -> Cosmos3TokenizedPrompt:
        chat = []
        if self.use_system_prompt:
            chat.append({"role": "system", "content": "You are a helpful assistant who will generate videos from a given prompt."})
        chat.append({"role": "user", "content": self._augment(prompt) if augment else prompt})
        ids = _flat_ids(self.tokenizer.apply_chat_template(chat, tokenize=True, add_generation_prompt=True))
        ids += [self.eos_token_id, self.vision_start_token_id]
        t = torch.tensor([ids], dtype=torch.long, device=device)
        return Cosmos3TokenizedPrompt(t, torch.ones_like(t))

    def tokenize_pair(self, prompt: str, negative_prompt: str | None = None, *, device="cpu"):
        neg = negative_prompt if negative_prompt is not None else (self._negative if self._negative is not None else cosmos3_default_negative_prompt())
        return self.tokenize(prompt, device=device, augment=True), self.tokenize(neg, device=device, augment=False)


@dataclass
class Cosmos3GenerationOutput:
    """Media of one generation request on the CPU: ``frames`` (T, H, W, 3) uint8 RGB, ``video`` as the engine returned
    it ([0, 1] floats), and for requests with sound the ``waveform`` in [-1, 1] with its ``sample_rate``. Fields can
    also be read by name like a dict (``out["frames"]``)."""

    frames: torch.Tensor
    video: torch.Tensor
    waveform: torch.Tensor | None = None
    sample_rate: int | None = None

    def __getitem__(self, key: str):
        if key not in ("frames", "video", "waveform", "sample_rate"):
            raise KeyError(key)
        return getattr(self, key)


class Cosmos3GenerationPostProcessor:
    """Output side of the generation plugin (its pixels are already VAE-decoded): tensors to the CPU, pixels to uint8
    frames, frames (and sound) into an mp4 through PyAV or into an ``.npz``."""

    def __init__(self, fps: float) -> None:
        self.fps = float(fps)

    @staticmethod
    def to_uint8_frames(video: torch.Tensor) -> torch.Tensor:
        """(1, 3, T, H, W) or (3, T, H, W) in [0, 1] -> (T, H, W, 3) uint8 of the first sample."""
        v = video[0] if video.dim() == 5 else video
        if v.dim() != 4 or v.shape[0] != 3:
            raise ValueError(f"a video is (1, 3, T, H, W) or (3, T, H, W), got {tuple(video.shape)}")
        return (v.float().clamp(0, 1) * 255.0).round().to(torch.uint8).permute(1, 2, 3, 0).contiguous().cpu()

    def postprocess(self, output) -> Cosmos3GenerationOutput:
        video, waveform, rate = (output["video"], output.get("sound"), output.get("sample_rate")) if isinstance(output, dict) else (output, None, None)
        if not isinstance(video, torch.Tensor):
            raise TypeError(f"expected a video tensor, got {type(video)!r}")
        wave = waveform.detach().clamp(-1.0, 1.0).float().cpu() if isinstance(waveform, torch.Tensor) else None
        return Cosmos3GenerationOutput(self.to_uint8_frames(video), video.detach().cpu(), wave, int(rate) if rate is not None else None)

    def save_mp4(self, output, path: str | Path, *, waveform: torch.Tensor | None = None, sample_rate: int | None = None,
                 crf: str = "18") -> Path:
        """H.264 (+ AAC when there is a waveform) through PyAV. ``output``: what :meth:`postprocess` returned, or bare
        frames with ``waveform`` / ``sample_rate`` beside them. Without PyAV this raises; :meth:`save_npz` needs nothing."""
        try:
            import av
        except ImportError as e:
            raise RuntimeError("writing mp4 needs the 'av' package; use save_npz for a dependency-free dump") from e
        if isinstance(output, Cosmos3GenerationOutput):
            frames, waveform, sample_rate = output.frames, output.waveform, output.sample_rate
        else:
            frames = output
        if waveform is not None and waveform.dim() == 3:
            waveform = waveform[0]
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        with av.open(str(path), mode="w") as c:
            vs = c.add_stream("h264", rate=round(self.fps))
            vs.height, vs.width, vs.pix_fmt = int(frames.shape[1]), int(frames.shape[2]), "yuv420p"
            vs.options = {"crf": str(crf)}
            aus = None
            if waveform is not None and sample_rate:
                aus = c.add_stream("aac", rate=int(sample_rate))
            for f in frames.numpy():
                for pkt in vs.encode(av.VideoFrame.from_ndarray(f, format="rgb24")):
                    c.mux(pkt)
            for pkt in vs.encode():
                c.mux(pkt)
            if aus is not None:
                af = av.AudioFrame.from_ndarray(waveform.numpy().astype("float32"), format="fltp",
                                                layout="stereo" if waveform.shape[0] == 2 else "mono")
                af.sample_rate = int(sample_rate)
                for pkt in aus.encode(af):
                    c.mux(pkt)
                for pkt in aus.encode():
                    c.mux(pkt)
        return path

    def save_npz(self, frames, path: str | Path, **extra) -> Path:
        if isinstance(frames, Cosmos3GenerationOutput):
            extra = {**({"waveform": frames.waveform, "sample_rate": frames.sample_rate} if frames.waveform is not None else {}), **extra}
            frames = frames.frames
        path = Path(path)
        np.savez_compressed(path, frames=frames.numpy(), fps=self.fps, **{k: (v.numpy() if hasattr(v, "numpy") else v) for k, v in extra.items()})
        return path


# ---------------------------------------------------------------- policy steps
def _to_rgb_uint8(value: Any) -> np.ndarray:
    """A path, PIL image, array or tensor -> ``(H, W, 3)`` uint8. Channel-first inputs are turned; float inputs are read
    as [0, 1], or as [-1, 1] when a value falls outside [0, 1]."""
    import PIL.Image

    if isinstance(value, (str, Path)):
        return np.asarray(PIL.Image.open(value).convert("RGB"))
    if isinstance(value, PIL.Image.Image):
        return np.asarray(value.convert("RGB"))
    if isinstance(value, torch.Tensor):
        value = value.detach().cpu().numpy() if value.dtype != torch.bfloat16 else value.detach().float().cpu().numpy()
    if not isinstance(value, np.ndarray):
        raise TypeError(f"an image is a path, a PIL image, an array or a tensor, not {type(value)!r}")
    arr = value
    if arr.ndim == 3 and arr.shape[0] in (3, 4) and arr.shape[-1] not in (3, 4):
        arr = np.transpose(arr, (1, 2, 0))
    if np.issubdtype(arr.dtype, np.floating):
        if arr.min() < 0.0 or arr.max() > 1.0:
            arr = np.clip(arr, -1.0, 1.0) * 0.5 + 0.5
        arr = (np.clip(arr, 0.0, 1.0) * 255.0).round().astype(np.uint8)
    return np.asarray(PIL.Image.fromarray(arr).convert("RGB"))


def resize_and_pad_action_image(image: Any, target_h: int, target_w: int) -> np.ndarray:
    """Observation frame -> ``(target_h, target_w, 3)`` uint8 the way the action variants were trained: shrink (never
    grow) with bicubic resampling until it fits, then fill to the right and below by reflection (by edge replication
    where a margin is as wide as the picture)."""
    import PIL.Image

    arr = _to_rgb_uint8(image)
    h, w = arr.shape[:2]
    scale = min(target_w / w, target_h / h, 1.0)
    rw, rh = max(1, int(scale * w + 0.5)), max(1, int(scale * h + 0.5))
    if (rw, rh) != (w, h):
        arr = np.asarray(PIL.Image.fromarray(arr).resize((rw, rh), PIL.Image.Resampling.BICUBIC))
    below, right = target_h - rh, target_w - rw
    if below == 0 and right == 0:
        return arr
    return np.pad(arr, ((0, below), (0, right), (0, 0)), mode="reflect" if below < rh and right < rw else "edge")


@ProcessorStepRegistry.register("cosmos3_image_preprocess_step")
class Cosmos3ImagePreprocessStep(ProcessorStep):
    """Observation frame(s) -> ``pixel_values`` (1, 3, T, H, W) in [-1, 1] and ``video_shape`` (T, H, W) in pixels.

    With ``image_size`` the target is the training bucket nearest to the first frame's aspect ratio at that height
    (:func:`resolve_target_size`) and ``meta_height`` / ``meta_width`` record the scaled size before padding; without it
    the target is ``height`` x ``width``. Every frame given is kept (one image: T = 1)."""

    def __init__(self, *, height: int, width: int, mode: str, image_size: int | None = None) -> None:
        self.height, self.width, self.mode = int(height), int(width), mode
        self.image_size = int(image_size) if image_size is not None else None

    def __call__(self, t: Transition) -> Transition:
        raw = t.get(IMAGES)
        if raw is None:
            raise ValueError("the image step needs 'images'")
        frames = list(raw) if isinstance(raw, (list, tuple)) else [raw]
        if self.image_size is not None:
            h0, w0 = _to_rgb_uint8(frames[0]).shape[:2]
            meta = (self.image_size, max(1, int(round(w0 * self.image_size / h0))))
            th, tw = resolve_target_size(h0, w0, self.image_size)
        else:
            th, tw = self.height, self.width
            meta = (th, tw)
        pix = [torch.from_numpy(resize_and_pad_action_image(f, th, tw).copy()).permute(2, 0, 1).float() / 127.5 - 1.0 for f in frames]
        out = dict(t)
        out[PIXEL_VALUES] = torch.stack(pix, dim=1)[None]
        out[VIDEO_SHAPE] = (len(pix), th, tw)
        out[META_HEIGHT], out[META_WIDTH] = meta
        return out

    def get_config(self):
        return {"height": self.height, "width": self.width, "mode": self.mode, "image_size": self.image_size}


@ProcessorStepRegistry.register("cosmos3_text_tokenize_step")
class Cosmos3TextTokenizeStep(ProcessorStep):
    """Task text -> ids of the conditional and the unconditional prompt.

    ``prompt_format="json"``: the structured action caption (:func:`cosmos3_action_json_caption`) with the padded frame
    size from ``video_shape``. ``"plain"``: the task with a duration / frame-rate sentence and a resolution sentence
    (the scaled size before padding) appended when ``append_metadata`` is set. The negative prompt is tokenised as it is.
    ``tokenizer`` takes a tokenizer object in place of a name to load (tests, offline use)."""

    def __init__(self, *, tokenizer_name_or_path: str | None = None, tokenizer: Any = None, negative_prompt: str = "",
                 append_metadata: bool = True, prompt_format: str = "plain", view_point: str = "ego_view", fps: float = 24.0,
                 num_frames: int = 17) -> None:
        if prompt_format not in ("plain", "json"):
            raise ValueError(f"prompt_format is 'plain' or 'json', not {prompt_format!r}")
        self.proc = Cosmos3Processor(tokenizer_name_or_path, tokenizer=tokenizer)
        self.tokenizer_name_or_path, self.negative_prompt, self.append_metadata = tokenizer_name_or_path, negative_prompt, bool(append_metadata)
        self.prompt_format, self.view_point, self.fps, self.num_frames = prompt_format, view_point, float(fps), int(num_frames)

    def _with_metadata(self, prompt: str, t: Transition) -> str:
        h, w = t.get(META_HEIGHT), t.get(META_WIDTH)
        if (h is None or w is None) and t.get(VIDEO_SHAPE) is not None:
            _, h, w = t[VIDEO_SHAPE]
        parts = [f"The video is {self.num_frames / self.fps:.1f} seconds long and is of {self.fps:.0f} FPS."]
        if h is not None and w is not None:
            parts.append(f"This video is of {h}x{w} resolution.")
        for sentence in parts:
            prompt += (" " if prompt.rstrip().endswith(".") else ". ") + sentence
        return prompt

    def __call__(self, t: Transition) -> Transition:
        task = t.get(TASK)
        if task is None:
            raise ValueError("the text step needs 'task'")
        if isinstance(task, (list, tuple)):
            task = task[0]
        if self.prompt_format == "json":
            shape = t.get(VIDEO_SHAPE)
            h, w = (shape[1], shape[2]) if shape is not None else (None, None)
            task = cosmos3_action_json_caption(task, view_point=self.view_point, num_frames=self.num_frames, fps=self.fps, height=h, width=w)
        elif self.append_metadata:
            task = self._with_metadata(task, t)
        pos, neg = self.proc.tokenize_pair(task, self.negative_prompt, device="cpu")
        out = dict(t)
        out[TEXT_IDS], out[TEXT_MASK], out[NEG_TEXT_IDS], out[NEG_TEXT_MASK] = pos.text_ids, pos.text_mask, neg.text_ids, neg.text_mask
        return out

    def get_config(self):
        return {"negative_prompt": self.negative_prompt, "append_metadata": self.append_metadata, "prompt_format": self.prompt_format,
                "view_point": self.view_point, "fps": self.fps, "num_frames": self.num_frames}


@ProcessorStepRegistry.register("cosmos3_action_pad_step")
class Cosmos3ActionPadStep(ProcessorStep):
    """Forward dynamics: conditioning actions -> (1, chunk, action_dim), the last action repeated up to the chunk length,
    channels zero-padded to the model width. Other modes carry no conditioning action."""

    def __init__(self, *, action_chunk_size: int, raw_action_dim: int, action_dim: int = 64, mode: str = "policy") -> None:
        self.action_chunk_size, self.raw_action_dim, self.action_dim, self.mode = int(action_chunk_size), int(raw_action_dim), int(action_dim), mode

    def __call__(self, t: Transition) -> Transition:
        out = dict(t)
        out[ACTION_CHUNK], out[RAW_ACTION_DIM] = self.action_chunk_size, self.raw_action_dim
        out.setdefault(MODE, self.mode)
        if self.mode != "forward_dynamics":
            out[COND_ACTION] = None
            return out
        a = t.get(COND_ACTION)
        if a is None:
            raise ValueError("forward_dynamics needs 'cond_action'")
        a = torch.as_tensor(np.asarray(a) if not isinstance(a, torch.Tensor) else a, dtype=torch.float32)
        if a.dim() == 3:
            a = a[0]
        n = self.action_chunk_size
        a = torch.cat([a, a[-1:].expand(n - a.shape[0], -1)]) if a.shape[0] < n else a[:n]
        padded = torch.zeros(n, self.action_dim)
        k = min(a.shape[-1], self.action_dim)
        padded[:, :k] = a[:, :k]
        out[COND_ACTION] = padded[None]
        return out

    def get_config(self):
        return {"action_chunk_size": self.action_chunk_size, "raw_action_dim": self.raw_action_dim, "action_dim": self.action_dim, "mode": self.mode}


@ProcessorStepRegistry.register("cosmos3_domain_resolve_step")
class Cosmos3DomainResolveStep(ProcessorStep):
    def __call__(self, t: Transition) -> Transition:
        if t.get(DOMAIN_ID) is None:
            raise ValueError("the domain step needs 'domain_id' (an embodiment name or an int)")
        out = dict(t)
        out[DOMAIN_ID] = resolve_domain_id(t[DOMAIN_ID])
        return out


@dataclass
class Cosmos3PolicyProcessedInputs:
    """What a ``Cosmos3ActionRequest`` is built from (``video_shape`` is in pixels: frames, height, width)."""

    pixel_values: torch.Tensor
    text_ids: torch.Tensor
    text_mask: torch.Tensor
    neg_text_ids: torch.Tensor
    neg_text_mask: torch.Tensor
    cond_action: torch.Tensor | None
    domain_id: int
    mode: str
    action_chunk: int
    raw_action_dim: int
    video_shape: tuple[int, int, int]
    cond_frame_indexes: tuple[int, ...] | None = None


_ACTION_NORMALIZATIONS = ("meanstd", "minmax", "quantile", "quantile_rot")


class Cosmos3PolicyProcessor(BaseModelProcessor):
    """Pre / post processing of the action variants. ``preprocess`` takes a dict with ``images`` (one frame or a list),
    ``task`` (or ``prompt``), for forward dynamics ``action`` (or ``cond_action``), optionally ``domain_name`` /
    ``domain_id`` and ``mode``. ``postprocess`` cuts the predicted chunk to the embodiment's action width and, when
    statistics were given (``action_stats_path``: a JSON file, or ``action_stats``: the same dict), maps it back to
    robot units. Arguments and output fields follow the reference
    (phyai-utils-tools/src/phyai_utils_tools/models/cosmos3/processor_cosmos3.py:326-560)."""

    def __init__(self, *, tokenizer_name_or_path: str | None = None, tokenizer: Any = None, height: int = 480, width: int = 832,
                 num_frames: int = 17, mode: str = "policy", domain_name: str | int = "agibotworld", action_chunk_size: int = 16,
                 raw_action_dim: int | None = None, action_dim: int = 64, negative_prompt: str = "", fps: float = 24.0,
                 image_size: int | None = None, append_metadata: bool = True, prompt_format: str = "plain", view_point: str = "ego_view",
                 cond_frame_indexes: tuple[int, ...] | None = None, action_stats_path: str | Path | None = None,
                 action_stats: dict | None = None, action_normalization: str = "minmax", device="cpu",
                 params_dtype: torch.dtype = torch.bfloat16) -> None:
        if action_normalization not in _ACTION_NORMALIZATIONS:
            raise ValueError(f"action_normalization is one of {_ACTION_NORMALIZATIONS}, not {action_normalization!r}")
        self.tokenizer_name_or_path, self.tokenizer = tokenizer_name_or_path, tokenizer
        self.height, self.width, self.num_frames, self.mode, self.domain_name = int(height), int(width), int(num_frames), mode, domain_name
        self.action_chunk_size, self.action_dim = int(action_chunk_size), int(action_dim)
        self.raw_action_dim = self._raw_action_dim(raw_action_dim, domain_name)
        self.negative_prompt, self.fps, self.append_metadata = negative_prompt, float(fps), bool(append_metadata)
        self.image_size = int(image_size) if image_size is not None else None
        self.prompt_format, self.view_point = prompt_format, view_point
        self.cond_frame_indexes = tuple(cond_frame_indexes) if cond_frame_indexes is not None else None
        self.action_normalization, self.device, self.params_dtype = action_normalization, device, params_dtype
        self._offset = self._span = None          # action = x * span + offset over the first len(offset) channels
        self._halved = False                      # min-max / quantile statistics map [-1, 1], mean / std map as they are
        if action_stats_path is not None:
            action_stats = json.loads(Path(action_stats_path).read_text())
            if not isinstance(action_stats, dict):
                raise ValueError(f"{action_stats_path}: action statistics must be a JSON object")
        if action_stats is not None:
            self._set_action_stats(action_stats)
        self.preprocessor, self.postprocessor = self.build_preprocessor(), self.build_postprocessor()

    @staticmethod
    def _raw_action_dim(given: int | None, domain_name: str | int) -> int:
        if given is None:
            return resolve_raw_action_dim(domain_name)
        given = int(given)
        if isinstance(domain_name, str):
            known = EMBODIMENT_TO_RAW_ACTION_DIM.get(domain_name.strip().lower())
            if known is not None and known != given:
                raise ValueError(f"raw_action_dim={given} conflicts with the {known} on record for {domain_name!r}")
        return given

    def _set_action_stats(self, stats: dict) -> None:
        block = stats.get("global_raw" if self.action_normalization == "quantile_rot" else "global", stats)
        f32 = lambda k: torch.tensor(block[k], dtype=torch.float32)  # noqa: E731
        if self.action_normalization == "meanstd":
            self._offset, self._span, self._halved = f32("mean"), f32("std").clamp(min=1e-8), False
        else:
            lo, hi = ("min", "max") if self.action_normalization == "minmax" else ("q01", "q99")
            self._offset = f32(lo)
            self._span, self._halved = (f32(hi) - self._offset).clamp(min=1e-6), True

    def denormalize_action(self, action: torch.Tensor) -> torch.Tensor:
        """Model units -> robot units over the channels the statistics cover (as it is when none were given)."""
        if self._offset is None:
            return action
        k = self._offset.shape[0]
        x = action[..., :k]
        off, span = self._offset.to(action.device), self._span.to(action.device)
        return (x + 1.0) / 2.0 * span + off if self._halved else x * span + off

    def build_preprocessor(self) -> ProcessorPipeline:
        steps = [Cosmos3ImagePreprocessStep(height=self.height, width=self.width, mode=self.mode, image_size=self.image_size),
                 # the caption's duration is that of the rollout (chunk + 1 frames), not of the observation
                 Cosmos3TextTokenizeStep(tokenizer_name_or_path=self.tokenizer_name_or_path, tokenizer=self.tokenizer,
                                         negative_prompt=self.negative_prompt, append_metadata=self.append_metadata,
                                         prompt_format=self.prompt_format, view_point=self.view_point, fps=self.fps,
                                         num_frames=self.action_chunk_size + 1),
                 Cosmos3ActionPadStep(action_chunk_size=self.action_chunk_size, raw_action_dim=self.raw_action_dim,
                                      action_dim=self.action_dim, mode=self.mode),
                 Cosmos3DomainResolveStep()]

        def to_t(raw: dict) -> Transition:
            first = lambda *keys, default=None: next((raw[k] for k in keys if raw.get(k) is not None), default)  # noqa: E731
            return {IMAGES: raw.get("images"), TASK: first("task", "prompt", default=""), COND_ACTION: first("action", "cond_action"),
                    DOMAIN_ID: first("domain_name", "domain_id", default=self.domain_name), MODE: raw.get("mode", self.mode)}

        def to_out(t: Transition) -> Cosmos3PolicyProcessedInputs:
            return Cosmos3PolicyProcessedInputs(t[PIXEL_VALUES], t[TEXT_IDS], t[TEXT_MASK], t[NEG_TEXT_IDS], t[NEG_TEXT_MASK],
                                                t.get(COND_ACTION), t[DOMAIN_ID], t[MODE], t[ACTION_CHUNK], t[RAW_ACTION_DIM],
                                                tuple(t[VIDEO_SHAPE]), self.cond_frame_indexes)
        return ProcessorPipeline(steps, "cosmos3_policy_preprocessor", to_transition=to_t, to_output=to_out)

    def build_postprocessor(self) -> ProcessorPipeline:
        return ProcessorPipeline([], "cosmos3_policy_postprocessor")

    def postprocess(self, output) -> dict[str, Any]:
        if isinstance(output, torch.Tensor):
            output = {"action": output}
        res: dict[str, Any] = {}
        if "action" in output:
            res["action"] = self.denormalize_action(output["action"][:, :, :self.raw_action_dim]).cpu()
        for k in ("pixels", "video"):
            if k in output:
                res[k] = output[k].cpu()
        return res


__all__ = ["Cosmos3Processor", "Cosmos3TokenizedPrompt", "Cosmos3GenerationOutput", "Cosmos3GenerationPostProcessor", "Cosmos3PolicyProcessor",
           "Cosmos3PolicyProcessedInputs", "Cosmos3ImagePreprocessStep", "Cosmos3TextTokenizeStep", "Cosmos3ActionPadStep",
           "Cosmos3DomainResolveStep", "EMBODIMENT_TO_DOMAIN_ID", "EMBODIMENT_TO_RAW_ACTION_DIM", "VIDEO_RES_SIZE_INFO",
           "DEFAULT_VIEWPOINT_TEMPLATES", "resolve_domain_id", "resolve_raw_action_dim", "get_vision_data_resolution",
           "find_closest_target_size", "resolve_target_size", "resize_and_pad_action_image", "aspect_ratio_str",
           "cosmos3_action_json_caption", "cosmos3_generation_caption", "cosmos3_default_negative_prompt"]
