"""Processor building blocks on CPU: image geometry, every normalisation mode and its inverse, the step registry, the
pipeline (adapters, step-through, reset), tokeniser and device / batch / rename / slice steps."""

import pytest
import torch

from phyai_b200.tools import processing as pp
from phyai_b200.tools.tokenizer import ByteTokenizer


# ------------------------------------------------------------------ images
@pytest.mark.parametrize("h,w,th,tw,inner,offset", [(100, 200, 224, 224, (112, 224), (56, 0)),     # wide: bars above and below
                                                     (200, 100, 224, 224, (224, 112), (0, 56)),     # tall: bars left and right
                                                     (448, 448, 224, 224, (224, 224), (0, 0)),      # same aspect: no bars
                                                     (30, 40, 15, 30, (15, 20), (0, 5))])
def test_resize_with_pad_keeps_the_aspect_ratio_and_centres(h, w, th, tw, inner, offset):
    img = torch.ones(2, 3, h, w)
    out = pp.resize_with_pad(img, th, tw, pad_value=-1.0)
    assert out.shape == (2, 3, th, tw)
    ih, iw = inner
    top, left = offset
    assert torch.allclose(out[:, :, top:top + ih, left:left + iw], torch.ones(2, 3, ih, iw))
    assert (out == -1).sum() == 2 * 3 * (th * tw - ih * iw)                                          # everything else is padding


def test_resize_with_pad_odd_remainder_dtypes_and_errors():
    out = pp.resize_with_pad(torch.ones(1, 1, 10, 10), 13, 10)                                       # three spare rows: 1 above, 2 below
    assert out[0, 0, :, 0].tolist() == [0.0] + [1.0] * 10 + [0.0] * 2
    u8 = torch.full((1, 3, 8, 16), 200, dtype=torch.uint8)
    out = pp.resize_with_pad(u8, 16, 16)
    assert out.dtype == torch.uint8 and out[0, 0, 8, 8] == 200 and out[0, 0, 0, 0] == 0
    same = torch.rand(1, 3, 16, 16)
    assert pp.resize_with_pad(same, 16, 16) is same                                                  # nothing to do: the input itself
    with pytest.raises(ValueError, match=r"expects \(B, C, H, W\)"):
        pp.resize_with_pad(torch.ones(3, 8, 8), 4, 4)
    with pytest.raises(ValueError, match="unsupported image dtype"):
        pp.resize_with_pad(torch.ones(1, 3, 8, 8, dtype=torch.int32), 4, 4)
    assert torch.equal(pp.normalize_pixels(torch.tensor([0.0, 0.5, 1.0])), torch.tensor([-1.0, 0.0, 1.0]))


def test_image_steps_take_lists_or_stacks_and_uint8():
    cams = [torch.full((2, 3, 10, 20), 255, dtype=torch.uint8), torch.zeros(2, 3, 20, 10, dtype=torch.uint8)]
    t = pp.ResizeWithPadStep(height=8, width=8)({pp.IMAGES: cams})
    assert t[pp.PIXEL_VALUES].shape == (2, 2, 3, 8, 8) and t[pp.PIXEL_VALUES].dtype == torch.uint8
    t = pp.NormalizeImageStep()(t)
    px = t[pp.PIXEL_VALUES]
    assert px.dtype == torch.float32 and px.max() == 1.0 and px.min() == -1.0                        # 255 -> 1, 0 / padding -> -1
    stacked = pp.ResizeWithPadStep(height=8, width=8)({pp.IMAGES: torch.rand(2, 3, 3, 8, 8)})
    assert stacked[pp.PIXEL_VALUES].shape == (2, 3, 3, 8, 8)
    assert pp.ResizeWithPadStep(4, 6, 0.5, "nearest").get_config() == {"height": 4, "width": 6, "pad_value": 0.5, "mode": "nearest"}
    # the reference's spelling: a square target and the expected camera / channel counts
    sq = pp.ResizeWithPadStep(target_size=8, num_images=2, num_channels=3)
    assert (sq.height, sq.width) == (8, 8) and torch.equal(sq({pp.IMAGES: cams})[pp.PIXEL_VALUES], pp.ResizeWithPadStep(8, 8)({pp.IMAGES: cams})[pp.PIXEL_VALUES])
    assert sq.get_config() == {"height": 8, "width": 8, "pad_value": 0.0, "mode": "bilinear", "num_images": 2, "num_channels": 3}
    for bad, msg in (([cams[0]], "expected 2 cameras"), ([cams[0], torch.zeros(2, 1, 4, 4, dtype=torch.uint8)], "has 1 channels"),
                     (torch.zeros(2, 3, 8, 8), "stacked images are"), ([cams[0], torch.zeros(3, 4, 4)], "camera 1 is")):
        with pytest.raises(ValueError, match=msg):
            sq({pp.IMAGES: bad})


# ------------------------------------------------------------------ normalisation
STATS = {"mean": [1.0, 2.0], "std": [2.0, 4.0], "min": [0.0, -2.0], "max": [2.0, 2.0], "q01": [0.5, 0.0], "q99": [1.5, 4.0],
         "q10": [0.8, 1.0], "q90": [1.2, 3.0]}


@pytest.mark.parametrize("mode,want", [("MEAN_STD", [[0.0, 0.0], [1.0, -0.5]]), ("MIN_MAX", [[0.0, 1.0], [2.0, 0.0]]),
                                       ("QUANTILES", [[0.0, 0.0], [4.0, -1.0]]), ("QUANTILE10", [[0.0, 0.0], [10.0, -2.0]]),
                                       ("IDENTITY", [[1.0, 2.0], [3.0, 0.0]])])
def test_every_normalisation_mode_and_its_inverse(mode, want):
    feats = {"observation.state": pp.PolicyFeature(pp.FeatureType.STATE, (2,))}
    kw = dict(features=feats, norm_map={pp.FeatureType.STATE: pp.NormalizationMode(mode)}, stats={"observation.state": STATS}, eps=0.0)
    x = torch.tensor([[1.0, 2.0], [3.0, 0.0]])
    y = pp.NormalizerStep(**kw)({pp.STATE: x.clone()})[pp.STATE]
    assert torch.allclose(y, torch.tensor(want), atol=1e-6)
    back = pp.UnnormalizerStep(**kw)({pp.STATE: y})[pp.STATE]
    assert torch.allclose(back, x, atol=1e-6)


def test_normaliser_leaves_padding_columns_and_refuses_narrow_tensors():
    feats = {"action": {"type": "ACTION", "shape": [2]}}                                              # the json form of a feature
    step = pp.NormalizerStep(features=feats, norm_map={"ACTION": "MEAN_STD"}, stats={"action": {"mean": [1.0, 1.0], "std": [1.0, 1.0]}}, eps=0.0)
    out = step({pp.ACTION: torch.tensor([[2.0, 3.0, 9.0, 9.0]])})[pp.ACTION]
    assert out.tolist() == [[1.0, 2.0, 9.0, 9.0]]                                                     # columns past the statistics pass through
    with pytest.raises(ValueError, match="smaller than the statistics"):
        step({pp.ACTION: torch.tensor([[2.0]])})
    assert step({pp.STATE: torch.ones(1, 2)})[pp.STATE].tolist() == [[1.0, 1.0]]                      # no statistics for it: untouched
    cfg = step.get_config()
    assert cfg["features"] == {"action": {"type": "ACTION", "shape": [2]}} and cfg["norm_map"] == {"ACTION": "MEAN_STD"}
    assert set(step.state_dict()) == {"action.mean", "action.std"}


def test_statistics_from_a_sidecar_unless_given_explicitly():
    feats = {"s": pp.PolicyFeature(pp.FeatureType.STATE, (1,))}
    late = pp.NormalizerStep(features=feats, norm_map={pp.FeatureType.STATE: pp.NormalizationMode.MEAN_STD})
    assert late({pp.STATE: torch.tensor([[5.0]])})[pp.STATE].item() == 5.0                            # nothing loaded yet
    late.load_state_dict({"s.mean": torch.tensor([1.0]), "s.std": torch.tensor([2.0])})
    assert late({pp.STATE: torch.tensor([[5.0]])})[pp.STATE].item() == pytest.approx(2.0)
    fixed = pp.NormalizerStep(features=feats, norm_map={pp.FeatureType.STATE: pp.NormalizationMode.MEAN_STD},
                              stats={"s": {"mean": [0.0], "std": [1.0]}})
    fixed.load_state_dict({"s.mean": torch.tensor([100.0]), "s.std": torch.tensor([1.0])})
    assert fixed({pp.STATE: torch.tensor([[5.0]])})[pp.STATE].item() == pytest.approx(5.0)            # the constructor's statistics win


# ------------------------------------------------------------------ registry and pipeline
def test_registry_names_duplicates_and_unknown_steps():
    @pp.ProcessorStepRegistry.register("test_only_double")
    class Double(pp.ProcessorStep):
        def __call__(self, t):
            t["x"] = t["x"] * 2
            return t

    try:
        assert pp.ProcessorStepRegistry.get("test_only_double") is Double and Double._registry_name == "test_only_double"
        assert pp.ProcessorStepRegistry.register("test_only_double")(Double) is Double               # the same class again: fine
        with pytest.raises(ValueError, match="already registered"):
            @pp.ProcessorStepRegistry.register("test_only_double")
            class Other(pp.ProcessorStep):
                def __call__(self, t):
                    return t
        assert "test_only_double" in pp.ProcessorStepRegistry.list()
    finally:
        pp.ProcessorStepRegistry.unregister("test_only_double")
    with pytest.raises(KeyError, match="unknown processor step 'test_only_double'"):
        pp.ProcessorStepRegistry.get("test_only_double")
    for name in ("resize_with_pad_step", "normalize_image_step", "normalizer_processor", "unnormalizer_processor", "tokenizer_processor",
                 "device_processor", "to_batch_processor", "rename_observations_processor", "slice_action_step"):
        assert name in pp.ProcessorStepRegistry.list()


def test_pipeline_adapters_step_through_and_reset():
    class Add(pp.ProcessorStep):
        def __init__(self, n):
            self.n, self.resets = n, 0

        def __call__(self, t):
            t["x"] = t["x"] + self.n
            return t

        def reset(self):
            self.resets += 1

    steps = [Add(1), Add(10)]
    pipe = pp.ProcessorPipeline(steps, name="adder", to_transition=lambda v: {"x": v}, to_output=lambda t: t["x"])
    assert pipe(5) == 16 and len(pipe) == 2 and pipe[1] is steps[1]
    assert [t["x"] for t in pipe.step_through(5)] == [5, 6, 16]                                       # the input, then after every step
    pipe.reset()
    assert [s.resets for s in steps] == [1, 1]
    assert pp.ProcessorPipeline()({"a": 1}) == {"a": 1}                                               # no steps, identity adapters


# ------------------------------------------------------------------ small steps
def test_tokeniser_step_pads_right_and_counts_real_tokens():
    step = pp.TokenizerStep(tokenizer=ByteTokenizer(), max_length=8)
    t = step({pp.PROMPT: ["ab", "abcdefghij"]})
    assert t[pp.INPUT_IDS].shape == (2, 8) and t[pp.INPUT_IDS].dtype == torch.long
    assert t[pp.LANG_LENS].tolist() == [3, 8]                                                         # bos + 2 bytes; truncated to 8
    assert t[pp.INPUT_IDS][0].tolist() == [1, ord("a") + 3, ord("b") + 3, 0, 0, 0, 0, 0]
    assert step({pp.TASK: "x"})[pp.INPUT_IDS].shape == (1, 8)                                         # falls back to the task string
    left = pp.TokenizerStep(tokenizer=ByteTokenizer(), max_length=4, padding_side="left")({pp.PROMPT: "a"})
    assert left[pp.INPUT_IDS][0].tolist() == [0, 0, 1, ord("a") + 3]
    with pytest.raises(pp.ProcessorStepError, match="needs a tokenizer"):
        pp.TokenizerStep()({pp.PROMPT: "a"})
    assert step.get_config()["max_length"] == 8 and ByteTokenizer().decode(t[pp.INPUT_IDS][0]) == "ab"


def test_device_batch_rename_and_slice_steps():
    t = pp.DeviceStep(device="cpu", float_dtype="bfloat16")({"a": torch.ones(2), "ids": torch.ones(2, dtype=torch.long),
                                                             "cams": [torch.ones(1)], "name": "x"})
    assert t["a"].dtype == torch.bfloat16 and t["ids"].dtype == torch.long and t["name"] == "x" and t["cams"][0].device.type == "cpu"
    b = pp.AddBatchDimensionStep()({pp.STATE: torch.ones(3), pp.IMAGES: [torch.ones(3, 4, 4)], pp.TASK: "go", pp.ACTION: torch.ones(2)})
    assert b[pp.STATE].shape == (1, 3) and b[pp.IMAGES][0].shape == (1, 3, 4, 4) and b[pp.TASK] == ["go"] and b[pp.ACTION].shape == (1, 2)
    same = pp.AddBatchDimensionStep()({pp.STATE: torch.ones(2, 3), pp.IMAGES: torch.ones(2, 3, 4, 4)})
    assert same[pp.STATE].shape == (2, 3) and same[pp.IMAGES].shape == (1, 2, 3, 4, 4)               # (n, C, H, W) gains the batch axis
    r = pp.RenameObservationsStep({"observation.images.top": "top", "absent": "x"})({"observation.images.top": 1, "other": 2})
    assert r == {"top": 1, "other": 2}
    s = pp.SliceActionStep(action_dim=2)({pp.ACTION: torch.arange(12.0).reshape(1, 3, 4)})
    assert s[pp.ACTION].shape == (1, 3, 2) and pp.SliceActionStep()({pp.ACTION: torch.ones(1, 4)})[pp.ACTION].shape == (1, 4)
