"""Pi0.5 pre/post-processing: images -> (B, n, C, 224, 224), state -> 256-bin tokens inside the prompt,
prompt -> ids; actions -> un-normalised, sliced to the robot's width.

Reference: phyai-utils-tools/src/phyai_utils_tools/models/pi05/{ops_pi05,steps_pi05,processor_pi05}.py.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np
import torch

from .processing import (ACTION, INPUT_IDS, LANG_LENS, PIXEL_VALUES, PROMPT, STATE, TASK, BaseModelProcessor, DeviceStep,
                         FeatureType, NormalizationMode, NormalizeImageStep, NormalizerStep, ProcessorPipeline, ProcessorStep,
                         ProcessorStepRegistry, ResizeWithPadStep, SliceActionStep, TokenizerStep, Transition, UnnormalizerStep)

STATE_NUM_BINS = 256
STATE_FEATURE, ACTION_FEATURE = "observation.state", "action"
PI05_DEFAULT_TOKENIZER_NAME = "google/paligemma-3b-pt-224"
PI05_NORM_MAP = {FeatureType.VISUAL: NormalizationMode.IDENTITY, FeatureType.STATE: NormalizationMode.QUANTILES,
                 FeatureType.ACTION: NormalizationMode.QUANTILES}
PRE_JSON, POST_JSON = "policy_preprocessor.json", "policy_postprocessor.json"


def discretize_state(state: torch.Tensor, num_bins: int = STATE_NUM_BINS) -> np.ndarray:
    """[-1, 1] -> bin index in [0, num_bins). Values above 1 land in the last bin; values below -1 give -1, as the
    binning of the reference does (phyai-utils-tools/src/phyai_utils_tools/models/pi05/ops_pi05.py:29-31): states are
    expected to be normalised into range before this step."""
    edges = np.linspace(-1.0, 1.0, num_bins + 1)[:-1]
    return np.digitize(state.detach().to(torch.float32).cpu().numpy(), bins=edges) - 1


def build_prompts(tasks: list[str], bins: np.ndarray) -> list[str]:
    if len(tasks) != len(bins):
        raise ValueError(f"{len(tasks)} tasks for {len(bins)} states")
    out = []
    for task, row in zip(tasks, bins):
        clean = task.strip().replace("_", " ").replace("\n", " ")
        out.append(f"Task: {clean}, State: {' '.join(str(int(b)) for b in row)};\nAction: ")
    return out


@ProcessorStepRegistry.register("pi05_prepare_state_tokenizer_processor_step")
@dataclass
class StateTokenizerPrepareStep(ProcessorStep):
    """Normalised state + task text -> the Pi0.5 prompt string (the state enters the model as text)."""

    max_state_dim: int = 32

    def __call__(self, t: Transition) -> Transition:
        state, tasks = t.get(STATE), t.get(TASK)
        if state is None or tasks is None:
            raise ValueError("the Pi0.5 prompt step needs 'state' and 'task'")
        if isinstance(tasks, str):
            tasks = [tasks]
        if state.dim() == 1:
            state = state[None]
        if state.shape[-1] < self.max_state_dim:
            state = torch.nn.functional.pad(state, (0, self.max_state_dim - state.shape[-1]))
        t[PROMPT] = build_prompts(list(tasks), discretize_state(state))
        return t

    def get_config(self):
        return {"max_state_dim": self.max_state_dim}


@dataclass
class PI05ProcessedInputs:
    """Fields of a ``PI05Request`` (noise is the engine's business)."""

    pixel_values: torch.Tensor
    input_ids: torch.Tensor
    lang_lens: torch.Tensor


def _features(stats: dict | None) -> dict:
    f = {}
    for name, kind in ((STATE_FEATURE, FeatureType.STATE), (ACTION_FEATURE, FeatureType.ACTION)):
        if stats and name in stats:
            width = len(next(iter(stats[name].values())))
            f[name] = {"type": kind.value, "shape": [width]}
    return f


class PI05Processor(BaseModelProcessor):
    def __init__(self, *, image_size: int = 224, num_images: int = 3, tokenizer_max_length: int = 200, action_dim: int | None = None,
                 tokenizer_name: str = PI05_DEFAULT_TOKENIZER_NAME, tokenizer: Any = None, dataset_stats: dict | None = None,
                 normalize_pixels: bool = False, image_pad_value: float = 0.0, device="cpu", params_dtype: torch.dtype = torch.bfloat16,
                 max_state_dim: int = 32) -> None:
        self.image_size, self.num_images, self.tokenizer_max_length = int(image_size), int(num_images), int(tokenizer_max_length)
        self.action_dim, self.tokenizer_name, self.dataset_stats = action_dim, tokenizer_name, dataset_stats
        self.normalize_pixels, self.image_pad_value = bool(normalize_pixels), float(image_pad_value)
        self.device, self.params_dtype, self.max_state_dim = device, params_dtype, max_state_dim
        if tokenizer is None:
            from .tokenizer import get_tokenizer

            tokenizer = get_tokenizer(tokenizer_name)
        self.tokenizer = tokenizer
        self.preprocessor, self.postprocessor = self.build_preprocessor(), self.build_postprocessor()

    def _dtype_name(self) -> str:
        return str(self.params_dtype).replace("torch.", "")

    def build_preprocessor(self) -> ProcessorPipeline:
        steps: list[ProcessorStep] = [ResizeWithPadStep(self.image_size, self.image_size, self.image_pad_value)]
        if self.normalize_pixels:
            steps.append(NormalizeImageStep())
        steps += [NormalizerStep(features=_features(self.dataset_stats), norm_map=PI05_NORM_MAP, stats=self.dataset_stats),
                  StateTokenizerPrepareStep(self.max_state_dim),
                  TokenizerStep(tokenizer=self.tokenizer, max_length=self.tokenizer_max_length, tokenizer_name=self.tokenizer_name),
                  DeviceStep(device=str(self.device), float_dtype=self._dtype_name())]
        return ProcessorPipeline(steps, "policy_preprocessor", to_output=lambda t: PI05ProcessedInputs(t[PIXEL_VALUES], t[INPUT_IDS], t[LANG_LENS]))

    def build_postprocessor(self) -> ProcessorPipeline:
        steps = [DeviceStep(device="cpu", float_dtype="float32"),
                 UnnormalizerStep(features=_features(self.dataset_stats), norm_map=PI05_NORM_MAP, stats=self.dataset_stats),
                 SliceActionStep(self.action_dim)]
        return ProcessorPipeline(steps, "policy_postprocessor", to_transition=lambda a: {ACTION: a}, to_output=lambda t: t[ACTION])

    def save_pretrained(self, directory: str | Path) -> None:
        self.preprocessor.save_pretrained(directory, config_filename=PRE_JSON)
        self.postprocessor.save_pretrained(directory, config_filename=POST_JSON)

    @classmethod
    def from_pretrained(cls, directory: str | Path, *, tokenizer: Any = None, device="cpu", params_dtype=torch.bfloat16, **kw) -> "PI05Processor":
        """Rebuild from a checkpoint's two processor jsons (statistics come from their sidecars)."""
        self = cls.__new__(cls)
        self.device, self.params_dtype, self.tokenizer = device, params_dtype, tokenizer
        sk = {"tokenizer_processor": {"tokenizer": tokenizer} if tokenizer is not None else {},
              "device_processor": {"device": str(device), "float_dtype": str(params_dtype).replace("torch.", "")}}
        pre = ProcessorPipeline.from_pretrained(directory, PRE_JSON, step_kwargs=sk)
        pre.to_output = lambda t: PI05ProcessedInputs(t[PIXEL_VALUES], t[INPUT_IDS], t[LANG_LENS])
        post = ProcessorPipeline.from_pretrained(directory, POST_JSON, step_kwargs={"device_processor": {"device": "cpu", "float_dtype": "float32"}})
        post.to_transition, post.to_output = (lambda a: {ACTION: a}), (lambda t: t[ACTION])
        self.preprocessor, self.postprocessor = pre, post
        return self


def make_pi05_processors(**kw) -> tuple[ProcessorPipeline, ProcessorPipeline]:
    p = PI05Processor(**kw)
    return p.preprocessor, p.postprocessor


__all__ = ["STATE_NUM_BINS", "discretize_state", "build_prompts", "StateTokenizerPrepareStep", "PI05ProcessedInputs", "PI05Processor",
           "make_pi05_processors", "PI05_NORM_MAP", "STATE_FEATURE", "ACTION_FEATURE"]
