"""Cosmos3 prompt, image and action processing for the generation and policy plugins.

* ``Cosmos3Processor``: chat-template tokenisation of the positive / negative prompt, with the
  duration / resolution metadata the model was trained to see appended to the positive one.
* ``Cosmos3GenerationPostProcessor``: pixels in [0, 1] -> uint8 frames (+ writers).
* ``Cosmos3PolicyProcessor``: observation image -> padded pixels, structured JSON caption -> ids,
  conditioning actions padded to the model width, embodiment name -> domain id; actions back to
  the robot's units.

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
                         Transition, resize_with_pad)

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
# training resolution buckets: tier -> aspect "w,h" -> (width, height)
VIDEO_RES_SIZE_INFO = {
    "256": {"1,1": (256, 256), "4,3": (320, 256), "3,4": (256, 320), "16,9": (320, 192), "9,16": (192, 320)},
    "480": {"1,1": (640, 640), "4,3": (736, 544), "3,4": (544, 736), "16,9": (832, 480), "9,16": (480, 832)},
    "704": {"1,1": (960, 960), "4,3": (1088, 832), "3,4": (832, 1088), "16,9": (1280, 704), "9,16": (704, 1280)},
    "768": {"1,1": (1024, 1024), "4,3": (1184, 880), "3,4": (880, 1184), "16,9": (1360, 768), "9,16": (768, 1360)},
    "1080": {"1,1": (1440, 1440), "4,3": (1664, 1248), "3,4": (1248, 1664), "16,9": (1920, 1080), "9,16": (1080, 1920)},
}
VIEWPOINT_FRAMING = {"ego": "first-person view from the robot's head camera", "wrist": "close-up view from the wrist camera",
                     "third_person": "fixed third-person view of the workspace"}


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


def find_closest_target_size(h: int, w: int, resolution: str | int) -> tuple[int, int]:
    """(height, width) of the training bucket of this tier whose aspect ratio is nearest to h:w."""
    tier = VIDEO_RES_SIZE_INFO.get(str(resolution))
    if tier is None:
        raise ValueError(f"unknown resolution tier {resolution!r}; known: {sorted(VIDEO_RES_SIZE_INFO)}")
    ratio = w / h
    bw, bh = min(tier.values(), key=lambda wh: abs(math.log((wh[0] / wh[1]) / ratio)))
    return bh, bw


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
    if VIEWPOINT_FRAMING.get(view_point):
        out["cinematography"] = {"framing": VIEWPOINT_FRAMING[view_point]}
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


def cosmos3_default_negative_prompt() -> str:
    """A structured description of what a bad clip looks like (used when the caller gives no negative prompt)."""
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
                 aspect_ratio: str | None = None, append_metadata: bool = True, negative_prompt: str | None = None) -> None:
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


class Cosmos3GenerationPostProcessor:
    def __init__(self, fps: float) -> None:
        self.fps = float(fps)

    @staticmethod
    def to_uint8_frames(video: torch.Tensor) -> torch.Tensor:
        """(B, 3, T, H, W) or (3, T, H, W) in [0, 1] -> (T, H, W, 3) uint8 of the first sample."""
        v = video[0] if video.dim() == 5 else video
        return (v.float().clamp(0, 1) * 255.0).round().to(torch.uint8).permute(1, 2, 3, 0).contiguous().cpu()

    def postprocess(self, output) -> dict[str, Any]:
        if isinstance(output, dict):
            res = {"frames": self.to_uint8_frames(output["video"]), "fps": self.fps}
            if "sound" in output:
                res["waveform"], res["sample_rate"] = output["sound"][0].float().cpu(), int(output["sample_rate"])
            return res
        return {"frames": self.to_uint8_frames(output), "fps": self.fps}

    def save_mp4(self, frames: torch.Tensor, path: str | Path, *, waveform: torch.Tensor | None = None, sample_rate: int | None = None) -> Path:
        """H.264 (+ AAC) through PyAV when it is installed; otherwise raises and ``save_npz`` is the portable writer."""
        try:
            import av
        except ImportError as e:
            raise RuntimeError("writing mp4 needs the 'av' package; use save_npz for a dependency-free dump") from e
        path = Path(path)
        with av.open(str(path), mode="w") as c:
            vs = c.add_stream("h264", rate=round(self.fps))
            vs.height, vs.width, vs.pix_fmt = int(frames.shape[1]), int(frames.shape[2]), "yuv420p"
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

    def save_npz(self, frames: torch.Tensor, path: str | Path, **extra) -> Path:
        path = Path(path)
        np.savez_compressed(path, frames=frames.numpy(), fps=self.fps, **{k: (v.numpy() if hasattr(v, "numpy") else v) for k, v in extra.items()})
        return path


# ---------------------------------------------------------------- policy steps
def _to_chw_float(img) -> torch.Tensor:
    """PIL image / (H, W, 3) uint8 array / (3, H, W) tensor -> (3, H, W) float in [0, 1]."""
    if isinstance(img, torch.Tensor):
        t = img
    else:
        t = torch.from_numpy(np.asarray(img))
    if t.dim() == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
        t = t.permute(2, 0, 1)
    return t.float() / 255.0 if t.dtype == torch.uint8 else t.float()


@ProcessorStepRegistry.register("cosmos3_image_preprocess_step")
class Cosmos3ImagePreprocessStep(ProcessorStep):
    """Observation image -> (1, 3, 1, H, W) in [-1, 1] at the training bucket nearest to its aspect ratio."""

    def __init__(self, *, resolution: str | int = "480", temporal: int = 4, spatial: int = 16, action_chunk_size: int = 32) -> None:
        self.resolution, self.temporal, self.spatial, self.action_chunk_size = str(resolution), int(temporal), int(spatial), int(action_chunk_size)

    def __call__(self, t: Transition) -> Transition:
        imgs = t[IMAGES]
        img = _to_chw_float(imgs[0] if isinstance(imgs, (list, tuple)) else imgs)
        h, w = img.shape[-2:]
        th, tw = find_closest_target_size(h, w, self.resolution)
        scale = min(th / h, tw / w)
        t[META_HEIGHT], t[META_WIDTH] = int(h * scale), int(w * scale)
        pix = resize_with_pad(img[None], th, tw)[0] * 2.0 - 1.0
        t[PIXEL_VALUES] = pix[None, :, None]
        frames = self.action_chunk_size + 1
        t[VIDEO_SHAPE] = ((frames - 1) // self.temporal + 1, th // self.spatial, tw // self.spatial)
        return t

    def get_config(self):
        return {"resolution": self.resolution, "temporal": self.temporal, "spatial": self.spatial, "action_chunk_size": self.action_chunk_size}


@ProcessorStepRegistry.register("cosmos3_text_tokenize_step")
class Cosmos3TextTokenizeStep(ProcessorStep):
    def __init__(self, *, tokenizer: Any = None, tokenizer_name: str | None = None, view_point: str = "ego", fps: float = 10.0,
                 action_chunk_size: int = 32, json_caption: bool = True, negative_prompt: str = "") -> None:
        self.proc = Cosmos3Processor(tokenizer_name, tokenizer=tokenizer, append_metadata=False)
        self.tokenizer_name, self.view_point, self.fps = tokenizer_name, view_point, float(fps)
        self.action_chunk_size, self.json_caption, self.negative_prompt = int(action_chunk_size), bool(json_caption), negative_prompt

    def __call__(self, t: Transition) -> Transition:
        task = t[TASK][0] if isinstance(t[TASK], (list, tuple)) else t[TASK]
        if self.json_caption:
            _, h, w = t[VIDEO_SHAPE]
            task = cosmos3_action_json_caption(task, view_point=self.view_point, num_frames=self.action_chunk_size + 1, fps=self.fps,
                                               height=h * 16, width=w * 16)
        pos, neg = self.proc.tokenize(task, augment=False), self.proc.tokenize(self.negative_prompt, augment=False)
        t[TEXT_IDS], t[TEXT_MASK], t[NEG_TEXT_IDS], t[NEG_TEXT_MASK] = pos.text_ids, pos.text_mask, neg.text_ids, neg.text_mask
        return t

    def get_config(self):
        return {"tokenizer_name": self.tokenizer_name, "view_point": self.view_point, "fps": self.fps,
                "action_chunk_size": self.action_chunk_size, "json_caption": self.json_caption, "negative_prompt": self.negative_prompt}


@ProcessorStepRegistry.register("cosmos3_action_pad_step")
class Cosmos3ActionPadStep(ProcessorStep):
    """Forward dynamics: conditioning actions -> (1, chunk, action_dim), last action repeated / zero channel padding."""

    def __init__(self, *, action_chunk_size: int, raw_action_dim: int, action_dim: int = 64, mode: str = "policy") -> None:
        self.action_chunk_size, self.raw_action_dim, self.action_dim, self.mode = int(action_chunk_size), int(raw_action_dim), int(action_dim), mode

    def __call__(self, t: Transition) -> Transition:
        t[ACTION_CHUNK], t[RAW_ACTION_DIM], t[MODE] = self.action_chunk_size, self.raw_action_dim, self.mode
        if self.mode != "forward_dynamics":
            t[COND_ACTION] = None
            return t
        a = t.get(COND_ACTION)
        if a is None:
            raise ValueError("forward_dynamics needs 'cond_action'")
        a = torch.as_tensor(np.asarray(a) if not isinstance(a, torch.Tensor) else a, dtype=torch.float32)
        if a.dim() == 3:
            a = a[0]
        n = self.action_chunk_size
        a = torch.cat([a, a[-1:].expand(n - a.shape[0], -1)]) if a.shape[0] < n else a[:n]
        out = torch.zeros(n, self.action_dim)
        k = min(a.shape[-1], self.action_dim)
        out[:, :k] = a[:, :k]
        t[COND_ACTION] = out[None]
        return t

    def get_config(self):
        return {"action_chunk_size": self.action_chunk_size, "raw_action_dim": self.raw_action_dim, "action_dim": self.action_dim, "mode": self.mode}


@ProcessorStepRegistry.register("cosmos3_domain_resolve_step")
class Cosmos3DomainResolveStep(ProcessorStep):
    def __call__(self, t: Transition) -> Transition:
        if t.get(DOMAIN_ID) is None:
            raise ValueError("the domain step needs 'domain_id' (an embodiment name or an int)")
        t[DOMAIN_ID] = resolve_domain_id(t[DOMAIN_ID])
        return t


@dataclass
class Cosmos3PolicyProcessedInputs:
    """Fields of a ``Cosmos3ActionRequest``."""

    text_ids: torch.Tensor
    text_mask: torch.Tensor
    neg_text_ids: torch.Tensor
    neg_text_mask: torch.Tensor
    video_shape: tuple[int, int, int]
    mode: str
    domain_id: int
    action_chunk: int
    raw_action_dim: int
    cond_video_pixels: torch.Tensor
    cond_action: torch.Tensor | None


class Cosmos3PolicyProcessor(BaseModelProcessor):
    def __init__(self, *, tokenizer: Any = None, tokenizer_name: str | None = None, domain: str | int = "bridge_orig_lerobot",
                 raw_action_dim: int | None = None, action_chunk_size: int = 32, action_dim: int = 64, mode: str = "policy",
                 resolution: str | int = "480", fps: float = 10.0, view_point: str = "ego", action_stats: dict | None = None) -> None:
        self.domain, self.mode, self.action_chunk_size, self.action_dim = domain, mode, int(action_chunk_size), int(action_dim)
        self.raw_action_dim = int(raw_action_dim) if raw_action_dim is not None else resolve_raw_action_dim(domain)
        self.tokenizer, self.tokenizer_name, self.resolution, self.fps, self.view_point = tokenizer, tokenizer_name, resolution, fps, view_point
        self.action_stats = {k: torch.as_tensor(v, dtype=torch.float32) for k, v in (action_stats or {}).items()}
        self.preprocessor, self.postprocessor = self.build_preprocessor(), self.build_postprocessor()

    def build_preprocessor(self) -> ProcessorPipeline:
        steps = [Cosmos3ImagePreprocessStep(resolution=self.resolution, action_chunk_size=self.action_chunk_size),
                 Cosmos3TextTokenizeStep(tokenizer=self.tokenizer, tokenizer_name=self.tokenizer_name, view_point=self.view_point,
                                         fps=self.fps, action_chunk_size=self.action_chunk_size),
                 Cosmos3ActionPadStep(action_chunk_size=self.action_chunk_size, raw_action_dim=self.raw_action_dim,
                                      action_dim=self.action_dim, mode=self.mode),
                 Cosmos3DomainResolveStep()]

        def to_t(raw: dict) -> Transition:
            return {IMAGES: raw["image"], TASK: raw["task"], DOMAIN_ID: raw.get("domain", self.domain), COND_ACTION: raw.get("cond_action")}

        def to_out(t: Transition) -> Cosmos3PolicyProcessedInputs:
            return Cosmos3PolicyProcessedInputs(t[TEXT_IDS], t[TEXT_MASK], t[NEG_TEXT_IDS], t[NEG_TEXT_MASK], tuple(t[VIDEO_SHAPE]), t[MODE],
                                                int(t[DOMAIN_ID]), int(t[ACTION_CHUNK]), int(t[RAW_ACTION_DIM]), t[PIXEL_VALUES], t[COND_ACTION])
        return ProcessorPipeline(steps, "cosmos3_policy_preprocessor", to_transition=to_t, to_output=to_out)

    def build_postprocessor(self) -> ProcessorPipeline:
        return ProcessorPipeline([], "cosmos3_policy_postprocessor")

    def denormalize_action(self, action: torch.Tensor) -> torch.Tensor:
        """[-1, 1] -> robot units with the embodiment's (q01, q99) or (min, max) statistics, when given."""
        s = self.action_stats
        a = action.float().cpu()
        for lo, hi in (("q01", "q99"), ("min", "max")):
            if lo in s and hi in s:
                k = s[lo].shape[-1]
                a = a.clone()
                a[..., :k] = (a[..., :k] + 1.0) / 2.0 * (s[hi] - s[lo]) + s[lo]
                return a
        if "mean" in s and "std" in s:
            k = s["mean"].shape[-1]
            a = a.clone()
            a[..., :k] = a[..., :k] * s["std"] + s["mean"]
        return a

    def postprocess(self, output) -> dict[str, Any]:
        action = output["action"] if isinstance(output, dict) else output
        res = {"action": self.denormalize_action(action[..., :self.raw_action_dim])}
        if isinstance(output, dict):
            res.update({k: v for k, v in output.items() if k != "action"})
        return res


__all__ = ["Cosmos3Processor", "Cosmos3TokenizedPrompt", "Cosmos3GenerationPostProcessor", "Cosmos3PolicyProcessor",
           "Cosmos3PolicyProcessedInputs", "Cosmos3ImagePreprocessStep", "Cosmos3TextTokenizeStep", "Cosmos3ActionPadStep",
           "Cosmos3DomainResolveStep", "EMBODIMENT_TO_DOMAIN_ID", "EMBODIMENT_TO_RAW_ACTION_DIM", "VIDEO_RES_SIZE_INFO",
           "resolve_domain_id", "resolve_raw_action_dim", "find_closest_target_size", "aspect_ratio_str",
           "cosmos3_action_json_caption", "cosmos3_generation_caption", "cosmos3_default_negative_prompt"]
