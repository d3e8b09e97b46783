"""Processing pipelines: generic steps, lerobot-format round trip, Pi0.5 / Pi0 / Cosmos3 processors."""

import json

import numpy as np
import pytest
import torch

from phyai_b200.tools import cosmos3 as c3
from phyai_b200.tools.pi0 import PI0Processor, PadStateStep
from phyai_b200.tools.pi05 import ACTION_FEATURE, STATE_FEATURE, PI05Processor, build_prompts, discretize_state
from phyai_b200.tools.processing import (ACTION, IMAGES, PIXEL_VALUES, PROMPT, STATE, TASK, NormalizerStep, ProcessorPipeline, ProcessorStepError,
                                         ProcessorStepRegistry, ResizeWithPadStep, UnnormalizerStep, resize_with_pad)
from phyai_b200.tools.tokenizer import ByteTokenizer


def test_resize_with_pad_geometry_and_dtypes():
    img = torch.rand(2, 3, 100, 200)
    out = resize_with_pad(img, 64, 64, pad_value=-1.0)
    assert out.shape == (2, 3, 64, 64) and torch.all(out[:, :, :16] == -1.0) and torch.all(out[:, :, 48:] == -1.0)
    assert float(out[:, :, 16:48].min()) >= 0.0
    u8 = (torch.rand(1, 3, 50, 50) * 255).to(torch.uint8)
    assert resize_with_pad(u8, 32, 48).dtype == torch.uint8 and resize_with_pad(u8, 50, 50) is u8
    with pytest.raises(ValueError):
        resize_with_pad(torch.rand(3, 8, 8), 4, 4)
    t = ResizeWithPadStep(32, 32)({IMAGES: [torch.rand(1, 3, 40, 20), torch.rand(1, 3, 32, 32)]})
    assert t[PIXEL_VALUES].shape == (1, 2, 3, 32, 32)


@pytest.mark.parametrize("mode", ["MEAN_STD", "MIN_MAX", "QUANTILES", "QUANTILE10"])
def test_normalizer_round_trip(mode):
    stats = {STATE_FEATURE: {"mean": [0.5, -1.0], "std": [2.0, 0.5], "min": [-1.0, -3.0], "max": [4.0, 1.0], "q01": [-0.5, -2.0],
                             "q99": [3.0, 0.5], "q10": [0.0, -1.5], "q90": [2.0, 0.0]}}
    feats = {STATE_FEATURE: {"type": "STATE", "shape": [2]}}
    fwd = NormalizerStep(features=feats, norm_map={"STATE": mode}, stats=stats)
    inv = UnnormalizerStep(features=feats, norm_map={"STATE": mode}, stats=stats)
    x = torch.tensor([[1.0, -0.5, 9.0]])                   # third channel is padding beyond the statistics: untouched
    y = fwd({STATE: x.clone()})[STATE]
    assert y[0, 2] == 9.0 and not torch.allclose(y[:, :2], x[:, :2])
    assert torch.allclose(inv({STATE: y})[STATE], x, atol=1e-5)
    if mode == "MIN_MAX":
        assert torch.allclose(fwd({STATE: torch.tensor([[-1.0, 1.0]])})[STATE], torch.tensor([[-1.0, 1.0]]), atol=1e-6)


def test_pipeline_save_load_lerobot_layout(tmp_path):
    stats = {ACTION_FEATURE: {"q01": [-1.0, -2.0], "q99": [1.0, 2.0]}, STATE_FEATURE: {"q01": [0.0] * 3, "q99": [1.0] * 3}}
    p = PI05Processor(tokenizer=ByteTokenizer(), dataset_stats=stats, action_dim=2, image_size=32, num_images=2, tokenizer_max_length=256, params_dtype=torch.float32)
    p.save_pretrained(tmp_path)
    cfg = json.loads((tmp_path / "policy_preprocessor.json").read_text())
    names = [s["registry_name"] for s in cfg["steps"]]
    # the lerobot-portable core only: the resize step (this package's, lerobot resizes inside the model) is not written
    assert names == ["normalizer_processor", "pi05_prepare_state_tokenizer_processor_step", "tokenizer_processor", "device_processor"]
    post_names = [s["registry_name"] for s in json.loads((tmp_path / "policy_postprocessor.json").read_text())["steps"]]
    assert post_names == ["unnormalizer_processor", "device_processor"]
    norm = cfg["steps"][0]
    assert norm["config"]["norm_map"]["STATE"] == "QUANTILES" and (tmp_path / norm["state_file"]).is_file() and "stats" not in norm["config"]
    assert cfg["steps"][1]["config"] == {} and cfg["steps"][2]["config"]["task_key"] == "task"
    q = PI05Processor.from_pretrained(tmp_path, tokenizer=ByteTokenizer(), params_dtype=torch.float32, image_size=32, num_images=2, action_dim=2)
    assert [type(s).__name__ for s in q.preprocessor.steps][:2] == ["ResizeWithPadStep", "NormalizerStep"] and q.tokenizer_max_length == 256
    raw = {IMAGES: [torch.rand(1, 3, 48, 64)] * 2, STATE: torch.tensor([[0.25, 0.5, 1.0]]), TASK: ["pick_up the\ncube"]}
    a, b = p.preprocess(dict(raw)), q.preprocess(dict(raw))
    assert torch.equal(a.input_ids, b.input_ids) and torch.equal(a.pixel_values, b.pixel_values) and a.pixel_values.shape == (1, 2, 3, 32, 32)
    text = ByteTokenizer().decode(a.input_ids[0, : int(a.lang_lens[0])])
    assert text.startswith("Task: pick up the cube, State: ") and text.endswith(";\nAction: ")
    act = torch.zeros(1, 4, 32)
    out = q.postprocess(act)
    assert out.shape == (1, 4, 2) and torch.allclose(out, torch.zeros(1, 4, 2), atol=1e-6)     # midpoint of (q01, q99)
    cfg["steps"].append({"registry_name": "no_such_step", "config": {}})
    (tmp_path / "broken.json").write_text(json.dumps(cfg))
    with pytest.raises(ProcessorStepError):
        ProcessorPipeline.from_pretrained(tmp_path, "broken.json", step_kwargs={"tokenizer_processor": {"tokenizer": ByteTokenizer()}})
    assert "normalizer_processor" in ProcessorStepRegistry.list()


def test_pi05_state_binning_and_prompt():
    edge = -1 + 2 / 256                                                       # the left edge of bin 1
    bins = discretize_state(torch.tensor([[-1.0, 0.0, 0.999, 1.0, 1.5, -3.0, edge, edge - 1e-4]]))
    assert bins.tolist() == [[0, 128, 255, 255, 255, -1, 1, 0]]             # above range: last bin; below range: -1
    assert discretize_state(torch.tensor([0.25], dtype=torch.bfloat16)).tolist() == [160]     # bf16 states convert cleanly
    assert discretize_state(torch.tensor([[-1.0, 0.99]]), num_bins=4).tolist() == [[0, 3]]
    assert build_prompts(["a_b"], np.array([[1, 2]])) == ["Task: a b, State: 1 2;\nAction: "]
    with pytest.raises(ValueError):
        build_prompts(["a", "b"], np.array([[1]]))


def test_pi0_processor_and_pad_state():
    p = PI0Processor(tokenizer=ByteTokenizer(), image_size=32, tokenizer_max_length=16, params_dtype=torch.float32, action_dim=7)
    out = p.preprocess({IMAGES: torch.rand(1, 3, 3, 32, 32), STATE: torch.ones(1, 5), TASK: "wipe"})
    assert out.state.shape == (1, 32) and out.state[0, 5:].abs().sum() == 0 and out.pixel_values.shape == (1, 3, 3, 32, 32)
    assert ByteTokenizer().decode(out.input_ids[0, : int(out.lang_lens[0])]) == "wipe\n"
    assert p.postprocess(torch.ones(1, 10, 32)).shape == (1, 10, 7)
    with pytest.raises(ValueError):
        PadStateStep(4)({STATE: torch.ones(1, 5)})


class FakeChatTokenizer(ByteTokenizer):
    eos_token_id = 2

    def convert_tokens_to_ids(self, tok):
        return 7

    def apply_chat_template(self, chat, tokenize=True, add_generation_prompt=True):
        text = "".join(f"<{m['role']}>{m['content']}" for m in chat) + "<assistant>"
        return [b + 3 for b in text.encode()]


def test_cosmos3_captions_and_tokenization():
    cap = c3.cosmos3_generation_caption("A robot arm", fps=24, num_frames=93, height=720, width=1280)
    assert cap == "A robot arm. The video is 3.9 seconds long and is of 24 FPS. This video is of 720x1280 resolution."
    j = json.loads(c3.cosmos3_generation_caption('{"scene": "lab"}', fps=24, num_frames=1, height=480, width=832, aspect_ratio="16,9"))
    assert j == {"scene": "lab", "resolution": {"H": 480, "W": 832}, "aspect_ratio": "16,9"}
    a = json.loads(c3.cosmos3_action_json_caption("open the drawer", view_point="ego_view", num_frames=33, fps=10, height=480, width=832))
    assert a["actions"] == [{"time": "0:00-0:03", "description": "open the drawer."}] and a["duration"] == "3s" and a["aspect_ratio"] == "16,9"
    assert c3.resolve_domain_id("LIBERO") == 5 and c3.resolve_domain_id(3) == 3 and c3.resolve_raw_action_dim("pusht") == 2
    with pytest.raises(ValueError):
        c3.resolve_domain_id("nope")
    with pytest.raises(ValueError):
        c3.resolve_raw_action_dim(4)
    assert c3.find_closest_target_size(480, 640, "480") == (736, 544) and c3.aspect_ratio_str(30, 20) == "3,2"      # (width, height)
    proc = c3.Cosmos3Processor(tokenizer=FakeChatTokenizer(), fps=24, num_frames=93, height=720, width=1280)
    pos, neg = proc.tokenize_pair("A robot arm")
    assert pos.text_ids.shape[0] == 1 and pos.text_ids[0, -2:].tolist() == [2, 7] and pos.text_mask.all()
    assert "resolution" in ByteTokenizer().decode(pos.text_ids[0]) and "artifacts" in ByteTokenizer().decode(neg.text_ids[0])
    assert "seconds long" not in ByteTokenizer().decode(neg.text_ids[0])


def test_cosmos3_policy_processor_and_postprocess(tmp_path):
    stats = tmp_path / "stats.json"
    stats.write_text(json.dumps({"global": {"q01": [-2.0, -4.0], "q99": [2.0, 4.0]}}))
    p = c3.Cosmos3PolicyProcessor(tokenizer=FakeChatTokenizer(), domain_name="pusht", mode="forward_dynamics", action_chunk_size=8,
                                  image_size=480, prompt_format="json", fps=10.0, action_stats_path=stats, action_normalization="quantile",
                                  cond_frame_indexes=(0,))
    img = (np.random.rand(96, 128, 3) * 255).astype("uint8")
    out = p.preprocess({"images": img, "task": "push the T", "cond_action": np.ones((5, 2), dtype="float32")})
    # a 4:3 frame scaled to 480 rows falls into the 480 tier, whose 4:3 bucket is 736 x 544; the frame is small, so it is
    # not enlarged: it sits in the top-left corner and the margins repeat its edge
    assert out.video_shape == (1, 544, 736) and out.pixel_values.shape == (1, 3, 1, 544, 736)
    assert -1.0 <= float(out.pixel_values.min()) and float(out.pixel_values.max()) <= 1.0
    corner = torch.from_numpy(img).permute(2, 0, 1).float() / 127.5 - 1.0
    assert torch.equal(out.pixel_values[0, :, 0, :96, :128], corner)
    assert torch.equal(out.pixel_values[0, :, 0, 300, :128], corner[:, -1]) and torch.equal(out.pixel_values[0, :, 0, :96, 500], corner[:, :, -1])
    assert out.domain_id == 4 and out.raw_action_dim == 2 and out.action_chunk == 8 and out.mode == "forward_dynamics"
    assert out.cond_frame_indexes == (0,)
    assert out.cond_action.shape == (1, 8, 64) and out.cond_action[0, 7, :2].tolist() == [1.0, 1.0] and out.cond_action[0, :, 2:].abs().sum() == 0
    text = ByteTokenizer().decode(out.text_ids[0])
    assert '"actions": [{"time": "0:00-0:01", "description": "push the T."}]' in text and '"resolution": {"H": 544, "W": 736}' in text
    assert "first-person perspective" in text                                                     # the default view point's sentence
    res = p.postprocess({"action": torch.zeros(1, 8, 64), "video": torch.zeros(1), "other": 1})
    assert res["action"].shape == (1, 8, 2) and torch.allclose(res["action"], torch.zeros(1, 8, 2)) and set(res) == {"action", "video"}
    assert torch.allclose(p.postprocess(torch.ones(1, 8, 64))["action"], torch.tensor([2.0, 4.0]).expand(1, 8, 2))
    plain = c3.Cosmos3PolicyProcessor(tokenizer=FakeChatTokenizer(), domain_name="libero", raw_action_dim=7, height=32, width=48, fps=8.0,
                                      action_chunk_size=15)
    got = plain.preprocess({"images": [torch.rand(3, 32, 48), torch.rand(3, 32, 48)], "prompt": "stack the blocks", "domain_id": 9})
    assert got.video_shape == (2, 32, 48) and got.cond_action is None and got.domain_id == 9 and got.mode == "policy"
    assert "stack the blocks. The video is 2.0 seconds long and is of 8 FPS. This video is of 32x48 resolution." in ByteTokenizer().decode(got.text_ids[0])
    assert plain.postprocess(torch.ones(1, 15, 64))["action"].shape == (1, 15, 7)                 # no statistics: model units
    with pytest.raises(ValueError, match="conflicts with the 2 on record"):
        c3.Cosmos3PolicyProcessor(tokenizer=FakeChatTokenizer(), domain_name="pusht", raw_action_dim=3)
    with pytest.raises(ValueError, match="action_normalization"):
        c3.Cosmos3PolicyProcessor(tokenizer=FakeChatTokenizer(), domain_name="pusht", action_normalization="zscore")
    post = c3.Cosmos3GenerationPostProcessor(fps=24)
    media = post.postprocess({"video": torch.rand(1, 3, 5, 16, 24), "sound": torch.randn(1, 2, 96) * 3, "sample_rate": 48000})
    frames = media.frames
    assert frames.shape == (5, 16, 24, 3) and frames.dtype == torch.uint8 and media["frames"] is frames and media.video.shape == (1, 3, 5, 16, 24)
    assert media.sample_rate == 48000 and float(media.waveform.abs().max()) <= 1.0                # the waveform is clamped to [-1, 1]
    f = post.save_npz(frames, tmp_path / "clip.npz")
    assert np.load(f)["frames"].shape == (5, 16, 24, 3)
    saved = np.load(post.save_npz(media, tmp_path / "clip2.npz"))
    assert saved["frames"].shape == (5, 16, 24, 3) and saved["waveform"].shape == (1, 2, 96) and int(saved["sample_rate"]) == 48000
    with pytest.raises(KeyError):
        media["fps"]


def test_pi05_processor_end_to_end_and_saved_pair(tmp_path):
    """Images resized, state normalised by quantiles and written into the prompt as bins, tokens right-padded; the action
    chunk comes back un-normalised and cut to the robot's width; a saved pair rebuilds the same pipelines."""
    from phyai_b200.tools.pi05 import PI05Processor, StateTokenizerPrepareStep, make_pi05_processors

    stats = {"observation.state": {"q01": [0.0, 0.0], "q99": [2.0, 4.0]}, "action": {"q01": [-1.0] * 3, "q99": [3.0] * 3}}
    p = PI05Processor(tokenizer=ByteTokenizer(), image_size=16, num_images=2, tokenizer_max_length=160, params_dtype=torch.float32, action_dim=3,
                      dataset_stats=stats, max_state_dim=4, pad_state=True)
    sample = {IMAGES: torch.rand(1, 2, 3, 8, 16), STATE: torch.tensor([[1.0, 4.0]]), TASK: "pick_up the\ncube "}
    out = p.preprocess(dict(sample))
    assert out.pixel_values.shape == (1, 2, 3, 16, 16) and out.input_ids.shape == (1, 160)
    text = ByteTokenizer().decode(out.input_ids[0, : int(out.lang_lens[0])])
    # state 1.0 of [0, 2] -> 0 -> bin 128; 4.0 of [0, 4] -> ~1 -> bin 255; two padding columns at 0 -> bin 128
    assert text == "Task: pick up the cube, State: 128 255 128 128;\nAction: "
    bare = PI05Processor(tokenizer=ByteTokenizer(), image_size=16, num_images=2, tokenizer_max_length=160, params_dtype=torch.float32, dataset_stats=stats)
    bare_text = ByteTokenizer().decode(bare.preprocess(dict(sample)).input_ids[0])
    assert "State: 128 255;" in bare_text                                                        # default: the bins of the state given, no padding
    act = p.postprocess(torch.zeros(1, 5, 32))
    assert act.shape == (1, 5, 3) and torch.allclose(act, torch.ones(1, 5, 3), atol=1e-5)        # 0 of [-1, 3] -> the middle, 1.0
    assert act.device.type == "cpu" and p.postprocess(torch.zeros(1, 5, 32, dtype=torch.bfloat16)).dtype == torch.bfloat16
    assert StateTokenizerPrepareStep()({TASK: "fold_it"})[PROMPT] == ["Task: fold it;\nAction: "]   # no state: the task alone
    with pytest.raises(ValueError, match="needs 'task'"):
        StateTokenizerPrepareStep()({STATE: torch.zeros(1, 2)})
    with pytest.raises(ValueError, match="expected 2 cameras, got 3"):
        p.preprocess({IMAGES: torch.rand(1, 3, 3, 8, 16), STATE: torch.zeros(1, 2), TASK: "x"})
    with pytest.raises(ValueError, match="has 1 channels, expected 3"):
        p.preprocess({IMAGES: torch.rand(1, 2, 1, 8, 16), STATE: torch.zeros(1, 2), TASK: "x"})
    p.save_pretrained(tmp_path)
    assert (tmp_path / "policy_preprocessor.json").is_file() and (tmp_path / "policy_postprocessor.json").is_file()
    q = PI05Processor.from_pretrained(tmp_path, tokenizer=ByteTokenizer(), params_dtype=torch.float32, image_size=16, num_images=2, action_dim=3)
    assert q.pad_state and q.max_state_dim == 4                                                  # padding is on: it is saved with the step
    again = q.preprocess(dict(sample))
    assert torch.equal(again.input_ids, out.input_ids) and torch.equal(again.pixel_values, out.pixel_values)
    assert torch.allclose(q.postprocess(torch.zeros(1, 5, 32)), act)
    pre, post = make_pi05_processors(tokenizer=ByteTokenizer(), image_size=16, tokenizer_max_length=32, params_dtype=torch.float32)
    assert pre.name == "pi05_preprocessor" and post.name == "pi05_postprocessor" and len(pre) == 5 and len(post) == 3


def test_pi0_saved_pair_and_prompt_step_names(tmp_path):
    from phyai_b200.tools.pi0 import Pi0NewLineProcessor, Pi0PromptPrepareStep

    stats = {"observation.state": {"mean": [1.0] * 5, "std": [2.0] * 5}, "action": {"mean": [0.5] * 7, "std": [2.0] * 7}}
    p = PI0Processor(tokenizer=ByteTokenizer(), image_size=16, tokenizer_max_length=16, params_dtype=torch.float32, action_dim=7,
                     dataset_stats=stats)
    out = p.preprocess({IMAGES: torch.rand(1, 3, 3, 16, 16), STATE: torch.full((1, 5), 3.0), TASK: "Wipe Table"})
    assert torch.allclose(out.state[0, :5], torch.ones(5), atol=1e-6) and out.state[0, 5:].abs().sum() == 0    # (3 - 1) / 2, then zero padding
    assert ByteTokenizer().decode(out.input_ids[0, : int(out.lang_lens[0])]) == "Wipe Table\n"                # case is kept
    assert torch.allclose(p.postprocess(torch.ones(1, 4, 32)), torch.full((1, 4, 7), 2.5), atol=1e-6)
    p.save_pretrained(tmp_path)
    q = PI0Processor.from_pretrained(tmp_path, tokenizer=ByteTokenizer(), params_dtype=torch.float32)
    again = q.preprocess({IMAGES: torch.rand(1, 3, 3, 16, 16), STATE: torch.full((1, 5), 3.0), TASK: "Wipe Table"})
    assert torch.equal(again.state, out.state) and torch.equal(again.input_ids, out.input_ids)
    assert Pi0PromptPrepareStep()({TASK: ["a\n", "b"]})[PROMPT] == ["a\n", "b\n"]
    assert Pi0NewLineProcessor()({TASK: "c"})[PROMPT] == ["c\n"]                                              # the name lerobot checkpoints use
    with pytest.raises(ValueError, match="needs 'task'"):
        Pi0PromptPrepareStep()({})
    with pytest.raises(TypeError, match="must be a tensor"):
        PadStateStep()({STATE: [1.0]})
