"""Pi0 pre/post-processing: the state stays a vector (padded to 32), the prompt is the task plus a newline.

Reference: phyai-utils-tools/src/phyai_utils_tools/models/pi0/{steps_pi0,processor_pi0}.py.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from .pi05 import ACTION_FEATURE, POST_JSON, PRE_JSON, STATE_FEATURE, _features
from .processing import (ACTION, INPUT_IDS, LANG_LENS, PIXEL_VALUES, PROMPT, STATE, TASK, BaseModelProcessor, DeviceStep, FeatureType,
                         NormalizationMode, NormalizeImageStep, NormalizerStep, ProcessorPipeline, ProcessorStep,
                         ProcessorStepRegistry, ResizeWithPadStep, SliceActionStep, TokenizerStep, Transition, UnnormalizerStep)

PI0_DEFAULT_TOKENIZER_NAME = "google/paligemma-3b-pt-224"
PI0_NORM_MAP = {FeatureType.VISUAL: NormalizationMode.IDENTITY, FeatureType.STATE: NormalizationMode.MEAN_STD,
                FeatureType.ACTION: NormalizationMode.MEAN_STD}


@ProcessorStepRegistry.register("pi0_prompt_prepare_step")
@dataclass
class Pi0PromptPrepareStep(ProcessorStep):
    def __call__(self, t: Transition) -> Transition:
        tasks = t.get(TASK)
        if tasks is None:
            raise ValueError("the Pi0 prompt step needs 'task'")
        if isinstance(tasks, str):
            tasks = [tasks]
        t[PROMPT] = [s if s.endswith("\n") else s + "\n" for s in tasks]
        return t


@ProcessorStepRegistry.register("pi0_new_line_processor")
@dataclass
class Pi0NewLineProcessor(Pi0PromptPrepareStep):
    """Name under which lerobot checkpoints save the same step."""


@ProcessorStepRegistry.register("pad_state_step")
@dataclass
class PadStateStep(ProcessorStep):
    max_state_dim: int = 32

    def __call__(self, t: Transition) -> Transition:
        s = t.get(STATE)
        if not isinstance(s, torch.Tensor):
            raise TypeError("'state' must be a tensor")
        if s.dim() == 1:
            s = s[None]
        if s.dim() != 2:
            raise ValueError(f"'state' must be (B, state_dim), got {tuple(s.shape)}")
        if s.shape[-1] > self.max_state_dim:
            raise ValueError(f"state_dim {s.shape[-1]} exceeds {self.max_state_dim}")
        t[STATE] = torch.nn.functional.pad(s, (0, self.max_state_dim - s.shape[-1]))
        return t

    def get_config(self):
        return {"max_state_dim": self.max_state_dim}


@dataclass
class PI0ProcessedInputs:
    pixel_values: torch.Tensor
    input_ids: torch.Tensor
    lang_lens: torch.Tensor
    state: torch.Tensor


def _is_vision_glue(step: Any) -> bool:
    return isinstance(step, (ResizeWithPadStep, NormalizeImageStep))


def _two_or_three(num_images: int) -> int:
    if int(num_images) not in (2, 3):
        raise ValueError(f"pi0 takes exactly 2 or 3 images, got {num_images}")
    return int(num_images)


class PI0Processor(BaseModelProcessor):
    """Pi0 pre / post processing in lerobot's conventions: cameras resized with padding and mapped to [-1, 1]
    (``normalize_pixels``, on by default), state and action normalised by mean / std, the state zero-padded to
    ``max_state_dim`` and handed over as a tensor, the task newline-terminated and tokenised to 48 tokens; the action
    chunk cut to ``action_dim``, un-normalised and returned on the CPU. ``save_pretrained`` leaves the resize / pixel
    steps out of the json; ``from_pretrained`` puts them back (and a state-padding step and an action cut where the files
    have none). Arguments and behaviour follow phyai-utils-tools/src/phyai_utils_tools/models/pi0/processor_pi0.py:80-300."""

    def __init__(self, *, image_size: int = 224, num_channels: int = 3, num_images: int = 3, tokenizer_max_length: int = 48,
                 max_state_dim: int = 32, action_dim: int | None = None, tokenizer_name: str = PI0_DEFAULT_TOKENIZER_NAME,
                 tokenizer: Any = None, dataset_stats: dict | None = None, normalize_pixels: bool = True, image_pad_value: float = 0.0,
                 device="cpu", params_dtype=torch.bfloat16) -> None:
        self.image_size, self.num_channels, self.num_images = int(image_size), int(num_channels), _two_or_three(num_images)
        self.tokenizer_max_length, self.max_state_dim, self.action_dim = int(tokenizer_max_length), int(max_state_dim), action_dim
        self.tokenizer_name, self.dataset_stats = tokenizer_name, dataset_stats
        self.normalize_pixels, self.image_pad_value, self.device, self.params_dtype = bool(normalize_pixels), float(image_pad_value), device, params_dtype
        if tokenizer is None:
            from .tokenizer import get_tokenizer

            tokenizer = get_tokenizer(tokenizer_name)
        self.tokenizer = tokenizer
        self.preprocessor, self.postprocessor = self.build_preprocessor(), self.build_postprocessor()

    @staticmethod
    def _out(t: Transition) -> PI0ProcessedInputs:
        return PI0ProcessedInputs(t[PIXEL_VALUES], t[INPUT_IDS], t[LANG_LENS], t[STATE])

    def _vision_steps(self) -> list[ProcessorStep]:
        steps: list[ProcessorStep] = [ResizeWithPadStep(self.image_size, self.image_size, self.image_pad_value, num_images=self.num_images,
                                                        num_channels=self.num_channels)]
        if self.normalize_pixels:
            steps.append(NormalizeImageStep())
        return steps

    def build_preprocessor(self) -> ProcessorPipeline:
        steps = self._vision_steps() + [
            NormalizerStep(features=_features(self.dataset_stats), norm_map=PI0_NORM_MAP, stats=self.dataset_stats, device=self.device),
            PadStateStep(self.max_state_dim), Pi0PromptPrepareStep(),
            TokenizerStep(tokenizer=self.tokenizer, max_length=self.tokenizer_max_length, tokenizer_name=self.tokenizer_name),
            DeviceStep(device=self.device, float_dtype=self.params_dtype)]
        return ProcessorPipeline(steps, "pi0_preprocessor", to_output=self._out)

    def build_postprocessor(self) -> ProcessorPipeline:
        steps = [SliceActionStep(self.action_dim),
                 UnnormalizerStep(features=_features(self.dataset_stats), norm_map=PI0_NORM_MAP, stats=self.dataset_stats, device=self.device),
                 DeviceStep(device="cpu")]
        return ProcessorPipeline(steps, "pi0_postprocessor", to_transition=lambda a: {ACTION: a}, to_output=lambda t: t[ACTION])

    def save_pretrained(self, directory: str | Path) -> None:
        ProcessorPipeline([s for s in self.preprocessor.steps if not _is_vision_glue(s)], "policy_preprocessor").save_pretrained(
            directory, config_filename=PRE_JSON)
        ProcessorPipeline(list(self.postprocessor.steps), "policy_postprocessor").save_pretrained(directory, config_filename=POST_JSON)

    @classmethod
    def from_pretrained(cls, directory: str | Path, *, tokenizer: Any = None, tokenizer_name: str = PI0_DEFAULT_TOKENIZER_NAME,
                        image_size: int = 224, num_channels: int = 3, num_images: int = 3, max_state_dim: int = 32,
                        action_dim: int | None = None, normalize_pixels: bool = True, image_pad_value: float = 0.0, device="cpu",
                        params_dtype=torch.bfloat16) -> "PI0Processor":
        if tokenizer is None:
            from .tokenizer import get_tokenizer

            tokenizer = get_tokenizer(tokenizer_name)
        self = cls.__new__(cls)
        self.image_size, self.num_channels, self.num_images = int(image_size), int(num_channels), _two_or_three(num_images)
        self.action_dim, self.tokenizer_name, self.tokenizer, self.dataset_stats = action_dim, tokenizer_name, tokenizer, None
        self.normalize_pixels, self.image_pad_value, self.device, self.params_dtype = bool(normalize_pixels), float(image_pad_value), device, params_dtype
        pre = ProcessorPipeline.from_pretrained(directory, PRE_JSON, step_kwargs={
            "tokenizer_processor": {"tokenizer": tokenizer}, "device_processor": {"device": device, "float_dtype": params_dtype},
            "normalizer_processor": {"device": device}})
        post_kw: dict[str, dict] = {"unnormalizer_processor": {"device": device}}
        if action_dim is not None:
            post_kw["slice_action_step"] = {"action_dim": action_dim}
        post = ProcessorPipeline.from_pretrained(directory, POST_JSON, step_kwargs=post_kw)
        self.tokenizer_max_length = next((s.max_length for s in pre.steps if isinstance(s, TokenizerStep)), 48)
        self.max_state_dim = next((s.max_state_dim for s in pre.steps if isinstance(s, PadStateStep)), int(max_state_dim))
        steps = [*self._vision_steps(), *[s for s in pre.steps if not _is_vision_glue(s)]]
        if not any(isinstance(s, PadStateStep) for s in steps):
            # behind the last normaliser (statistics cover the real state width), else in front of the prompt / tokenizer steps
            after_norm = [i + 1 for i, s in enumerate(steps) if isinstance(s, NormalizerStep)]
            before_text = [i for i, s in enumerate(steps) if isinstance(s, (Pi0PromptPrepareStep, TokenizerStep))]
            at = after_norm[-1] if after_norm else (before_text[0] if before_text else len(steps))
            steps.insert(at, PadStateStep(self.max_state_dim))
        pre.steps, pre.name, pre.to_output = steps, "pi0_preprocessor", cls._out
        if not any(isinstance(s, SliceActionStep) for s in post.steps):
            post.steps = [SliceActionStep(action_dim), *post.steps]
        post.name, post.to_transition, post.to_output = "pi0_postprocessor", (lambda a: {ACTION: a}), (lambda t: t[ACTION])
        self.preprocessor, self.postprocessor = pre, post
        return self


def make_pi0_processors(**kw) -> tuple[ProcessorPipeline, ProcessorPipeline]:
    p = PI0Processor(**kw)
    return p.preprocessor, p.postprocessor


__all__ = ["Pi0PromptPrepareStep", "Pi0NewLineProcessor", "PadStateStep", "PI0ProcessedInputs", "PI0Processor", "make_pi0_processors", "PI0_NORM_MAP",
           "PI0_DEFAULT_TOKENIZER_NAME",
           "STATE_FEATURE", "ACTION_FEATURE"]
