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


class PI0Processor(BaseModelProcessor):
    def __init__(self, *, image_size: int = 224, num_images: int = 3, tokenizer_max_length: int = 48, max_state_dim: int = 32,
                 action_dim: int | None = None, tokenizer_name: str = "google/paligemma-3b-pt-224", tokenizer: Any = None,
                 dataset_stats: dict | None = None, normalize_pixels: bool = False, device="cpu", params_dtype=torch.bfloat16) -> None:
        self.image_size, self.num_images, self.tokenizer_max_length = image_size, num_images, tokenizer_max_length
        self.max_state_dim, self.action_dim, self.dataset_stats = max_state_dim, action_dim, dataset_stats
        self.normalize_pixels, self.device, self.params_dtype, self.tokenizer_name = normalize_pixels, device, params_dtype, tokenizer_name
        if tokenizer is None:
            from .tokenizer import get_tokenizer

            tokenizer = get_tokenizer(tokenizer_name)
        self.tokenizer = tokenizer
        self.preprocessor, self.postprocessor = self.build_preprocessor(), self.build_postprocessor()

    @staticmethod
    def _out(t: Transition) -> PI0ProcessedInputs:
        return PI0ProcessedInputs(t[PIXEL_VALUES], t[INPUT_IDS], t[LANG_LENS], t[STATE])

    def build_preprocessor(self) -> ProcessorPipeline:
        steps: list[ProcessorStep] = [ResizeWithPadStep(self.image_size, self.image_size)]
        if self.normalize_pixels:
            steps.append(NormalizeImageStep())
        steps += [NormalizerStep(features=_features(self.dataset_stats), norm_map=PI0_NORM_MAP, stats=self.dataset_stats),
                  PadStateStep(self.max_state_dim), Pi0PromptPrepareStep(),
                  TokenizerStep(tokenizer=self.tokenizer, max_length=self.tokenizer_max_length, tokenizer_name=self.tokenizer_name),
                  DeviceStep(device=str(self.device), float_dtype=str(self.params_dtype).replace("torch.", ""))]
        return ProcessorPipeline(steps, "policy_preprocessor", to_output=self._out)

    def build_postprocessor(self) -> ProcessorPipeline:
        steps = [DeviceStep(device="cpu", float_dtype="float32"),
                 UnnormalizerStep(features=_features(self.dataset_stats), norm_map=PI0_NORM_MAP, stats=self.dataset_stats),
                 SliceActionStep(self.action_dim)]
        return ProcessorPipeline(steps, "policy_postprocessor", to_transition=lambda a: {ACTION: a}, to_output=lambda t: t[ACTION])

    def save_pretrained(self, directory: str | Path) -> None:
        self.preprocessor.save_pretrained(directory, config_filename=PRE_JSON)
        self.postprocessor.save_pretrained(directory, config_filename=POST_JSON)

    @classmethod
    def from_pretrained(cls, directory: str | Path, *, tokenizer: Any = None, device="cpu", params_dtype=torch.bfloat16) -> "PI0Processor":
        self = cls.__new__(cls)
        self.device, self.params_dtype, self.tokenizer = device, params_dtype, tokenizer
        sk = {"tokenizer_processor": {"tokenizer": tokenizer} if tokenizer is not None else {},
              "device_processor": {"device": str(device), "float_dtype": str(params_dtype).replace("torch.", "")}}
        self.preprocessor = ProcessorPipeline.from_pretrained(directory, PRE_JSON, step_kwargs=sk, to_output=cls._out)
        self.postprocessor = ProcessorPipeline.from_pretrained(
            directory, POST_JSON, step_kwargs={"device_processor": {"device": "cpu", "float_dtype": "float32"}},
            to_transition=lambda a: {ACTION: a}, to_output=lambda t: t[ACTION])
        return self


__all__ = ["Pi0PromptPrepareStep", "Pi0NewLineProcessor", "PadStateStep", "PI0ProcessedInputs", "PI0Processor", "PI0_NORM_MAP",
           "STATE_FEATURE", "ACTION_FEATURE"]
