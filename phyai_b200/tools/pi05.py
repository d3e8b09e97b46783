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
    """Normalised state + task text -> the Pi0.5 prompt string (the state enters the model as text). Without a state the
    prompt carries the task alone. ``pad_state`` first pads the state with zeros to ``max_state_dim`` (lerobot's
    convention: the prompt then always lists that many bins); off by default, as in the reference
    (phyai-utils-tools/src/phyai_utils_tools/models/pi05/steps_pi05.py:30-68), whose prompt lists the bins of the state
    it is given. Like lerobot's step of this name it saves no configuration unless padding is on."""

    num_bins: int = STATE_NUM_BINS
    max_state_dim: int = 32
    pad_state: bool = False

    def __call__(self, t: Transition) -> Transition:
        tasks = t.get(TASK)
        if tasks is None:
            raise ValueError("the Pi0.5 prompt step needs 'task'")
        if isinstance(tasks, str):
            tasks = [tasks]
        out = dict(t)
        state = t.get(STATE)
        if state is None:
            out[PROMPT] = [f"Task: {s.strip().replace('_', ' ').replace(chr(10), ' ')};\nAction: " for s in tasks]
            return out
        if state.dim() == 1:
            state = state[None]
        if self.pad_state and state.shape[-1] < self.max_state_dim:
            state = torch.nn.functional.pad(state, (0, self.max_state_dim - state.shape[-1]))
        out[PROMPT] = build_prompts(list(tasks), discretize_state(state, self.num_bins))
        return out

    def get_config(self):
        return {"pad_state": True, "max_state_dim": self.max_state_dim} if self.pad_state else {}


@dataclass
class PI05ProcessedInputs:
    """Fields of a ``PI05Request`` (noise is the engine's business)."""

    pixel_values: torch.Tensor
    input_ids: torch.Tensor
    lang_lens: torch.Tensor


def _features(stats: dict | None) -> dict:
    return {name: {"type": kind.value, "shape": []} for name, kind in ((STATE_FEATURE, FeatureType.STATE), (ACTION_FEATURE, FeatureType.ACTION))
            if stats and name in stats}


def _is_vision_glue(step: Any) -> bool:
    """Steps that are this package's, not part of a lerobot processor json (lerobot resizes inside the model)."""
    return isinstance(step, (ResizeWithPadStep, NormalizeImageStep))


class PI05Processor(BaseModelProcessor):
    """Pi0.5 pre / post processing: cameras resized with padding (optionally to [-1, 1]), state and action normalised by
    the dataset statistics (quantiles; none given: identity), the state written into the prompt as bins, tokens padded to
    ``tokenizer_max_length``; the action chunk un-normalised, cut to ``action_dim`` and returned on the CPU.

    ``save_pretrained`` writes the lerobot-portable core (``policy_preprocessor.json`` / ``policy_postprocessor.json``
    with the statistics beside them): the resize / pixel steps and the action cut are rebuilt from arguments by
    ``from_pretrained``, which therefore also loads the processor files of a lerobot checkpoint. Arguments and behaviour
    follow phyai-utils-tools/src/phyai_utils_tools/models/pi05/processor_pi05.py:101-335."""

    def __init__(self, *, image_size: int = 224, num_channels: int = 3, num_images: int = 3, tokenizer_max_length: int = 200,
                 action_dim: int | None = None, tokenizer_name: str = PI05_DEFAULT_TOKENIZER_NAME, tokenizer: Any = None,
                 dataset_stats: dict | None = None, normalize_pixels: bool = False, image_pad_value: float = 0.0, device="cpu",
                 params_dtype: torch.dtype = torch.bfloat16, pad_state: bool = False, max_state_dim: int = 32) -> None:
        self.image_size, self.num_channels, self.num_images = int(image_size), int(num_channels), int(num_images)
        self.tokenizer_max_length, self.action_dim, self.tokenizer_name = int(tokenizer_max_length), action_dim, tokenizer_name
        self.dataset_stats, self.normalize_pixels, self.image_pad_value = dataset_stats, bool(normalize_pixels), float(image_pad_value)
        self.device, self.params_dtype, self.pad_state, self.max_state_dim = device, params_dtype, bool(pad_state), int(max_state_dim)
        if tokenizer is None:
            from .tokenizer import get_tokenizer

            tokenizer = get_tokenizer(tokenizer_name)
        self.tokenizer = tokenizer
        self.preprocessor, self.postprocessor = self.build_preprocessor(), self.build_postprocessor()

    @staticmethod
    def _inputs(t: Transition) -> PI05ProcessedInputs:
        return PI05ProcessedInputs(t[PIXEL_VALUES], t[INPUT_IDS], t[LANG_LENS])

    def _vision_steps(self) -> list[ProcessorStep]:
        steps: list[ProcessorStep] = [ResizeWithPadStep(self.image_size, self.image_size, self.image_pad_value, num_images=self.num_images,
                                                        num_channels=self.num_channels)]
        if self.normalize_pixels:
            steps.append(NormalizeImageStep())
        return steps

    def build_preprocessor(self) -> ProcessorPipeline:
        steps = self._vision_steps() + [
            NormalizerStep(features=_features(self.dataset_stats), norm_map=PI05_NORM_MAP, stats=self.dataset_stats, device=self.device),
            StateTokenizerPrepareStep(max_state_dim=self.max_state_dim, pad_state=self.pad_state),
            TokenizerStep(tokenizer=self.tokenizer, max_length=self.tokenizer_max_length, tokenizer_name=self.tokenizer_name),
            DeviceStep(device=self.device, float_dtype=self.params_dtype)]
        return ProcessorPipeline(steps, "pi05_preprocessor", to_output=self._inputs)

    def build_postprocessor(self) -> ProcessorPipeline:
        steps = [UnnormalizerStep(features=_features(self.dataset_stats), norm_map=PI05_NORM_MAP, stats=self.dataset_stats, device=self.device),
                 SliceActionStep(self.action_dim), DeviceStep(device="cpu")]
        return ProcessorPipeline(steps, "pi05_postprocessor", to_transition=lambda a: {ACTION: a}, to_output=lambda t: t[ACTION])

    def save_pretrained(self, directory: str | Path) -> None:
        ProcessorPipeline([s for s in self.preprocessor.steps if not _is_vision_glue(s)], "policy_preprocessor").save_pretrained(
            directory, config_filename=PRE_JSON)
        ProcessorPipeline([s for s in self.postprocessor.steps if not isinstance(s, SliceActionStep)], "policy_postprocessor").save_pretrained(
            directory, config_filename=POST_JSON)

    @classmethod
    def from_pretrained(cls, directory: str | Path, *, tokenizer: Any = None, tokenizer_name: str = PI05_DEFAULT_TOKENIZER_NAME,
                        image_size: int = 224, num_channels: int = 3, num_images: int = 3, action_dim: int | None = None,
                        normalize_pixels: bool = False, image_pad_value: float = 0.0, device="cpu",
                        params_dtype: torch.dtype = torch.bfloat16) -> "PI05Processor":
        """Rebuild from a checkpoint's two processor jsons (statistics come from their sidecars). The tokenizer object and
        the model's device are injected into the steps a json cannot carry; the postprocessor keeps the device the
        checkpoint names (actions return to the host). Resize / pixel steps go in front and the action cut behind
        unless the files already hold them."""
        if tokenizer is None:
            from .tokenizer import get_tokenizer

            tokenizer = get_tokenizer(tokenizer_name)
        self = cls.__new__(cls)
        self.image_size, self.num_channels, self.num_images = int(image_size), int(num_channels), int(num_images)
        self.action_dim, self.tokenizer_name, self.tokenizer, self.dataset_stats = action_dim, tokenizer_name, tokenizer, None
        self.normalize_pixels, self.image_pad_value = bool(normalize_pixels), float(image_pad_value)
        self.device, self.params_dtype = device, params_dtype
        pre = ProcessorPipeline.from_pretrained(directory, PRE_JSON, step_kwargs={
            "tokenizer_processor": {"tokenizer": tokenizer}, "device_processor": {"device": device}})
        post = ProcessorPipeline.from_pretrained(directory, POST_JSON, step_kwargs={"unnormalizer_processor": {"device": device}})
        self.tokenizer_max_length = next((s.max_length for s in pre.steps if isinstance(s, TokenizerStep)), 200)
        prep = next((s for s in pre.steps if isinstance(s, StateTokenizerPrepareStep)), None)
        self.pad_state, self.max_state_dim = (prep.pad_state, prep.max_state_dim) if prep is not None else (False, 32)
        if not any(_is_vision_glue(s) for s in pre.steps):
            pre.steps = [*self._vision_steps(), *pre.steps]
        if not any(isinstance(s, SliceActionStep) for s in post.steps):
            post.steps = [*post.steps, SliceActionStep(action_dim)]
        pre.name, pre.to_output = "pi05_preprocessor", cls._inputs
        post.name, post.to_transition, post.to_output = "pi05_postprocessor", (lambda a: {ACTION: a}), (lambda t: t[ACTION])
        self.preprocessor, self.postprocessor = pre, post
        return self


def make_pi05_processors(**kw) -> tuple[ProcessorPipeline, ProcessorPipeline]:
    p = PI05Processor(**kw)
    return p.preprocessor, p.postprocessor


__all__ = ["STATE_NUM_BINS", "discretize_state", "build_prompts", "StateTokenizerPrepareStep", "PI05ProcessedInputs", "PI05Processor",
           "make_pi05_processors", "PI05_NORM_MAP", "STATE_FEATURE", "ACTION_FEATURE"]
