"""This package against the unmodified reference installed under ``baseline/_ref``, piece by piece on CPU: the parts
of the reference that import and run without a GPU (sampler, rotary tables and position ids, prompt and bucket helpers,
state binning, image and normalisation steps). Skipped where the reference is not installed."""

import importlib
import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
pytestmark = pytest.mark.skipif(not (REF / "phyai").is_dir(), reason="the reference is not installed under baseline/_ref")


@pytest.fixture()
def ref():
    """``ref("phyai.x.y")`` imports a module of the reference; its folder is on the path only inside the test."""
    sys.path.insert(0, str(REF))
    try:
        yield importlib.import_module
    finally:
        sys.path.remove(str(REF))


@pytest.mark.parametrize("karras,shift,steps", [(True, 1.0, 8), (False, 1.0, 5), (False, 5.0, 12), (True, 3.0, 2), (False, 1.0, 1)])
def test_unipc_trajectory(ref, karras, shift, steps):
    from phyai_b200.models.cosmos3 import UniPCMultistepSampler

    theirs = ref("phyai.models.cosmos3.sampler_unipc").UniPCMultistepSampler(flow_shift=shift, use_karras_sigmas=karras)
    ours = UniPCMultistepSampler(flow_shift=shift, use_karras_sigmas=karras)
    theirs.set_timesteps(steps)
    ours.set_timesteps(steps)
    assert torch.allclose(ours.timesteps.float(), theirs.timesteps.float()) and torch.allclose(ours.sigmas.float(), theirs.sigmas.float(), atol=1e-6)
    g = torch.Generator().manual_seed(steps)
    xa = xb = torch.randn(2, 4, 3, 5, generator=g, dtype=torch.float64)
    w = torch.randn(5, 5, generator=g, dtype=torch.float64) * 0.3
    for t in theirs.timesteps:
        va, vb = torch.tanh(xa @ w) + 0.1 * xa, torch.tanh(xb @ w) + 0.1 * xb          # a smooth stand-in for the model
        xa, xb = theirs.step(va, t, xa), ours.step(vb, t, xb)
        # the reference holds its sigmas and coefficients in fp32 tensors, this package in Python floats
        assert torch.allclose(xa, xb, atol=2e-5, rtol=2e-5), (float(t), (xa - xb).abs().max())
    assert ours.step_index == theirs.step_index == steps


def test_position_ids_and_interleaved_rotary_tables(ref):
    from phyai_b200.layers.rotary_embedding import MRotaryEmbedding
    from phyai_b200.models.cosmos3 import modeling_cosmos3 as mine

    theirs = ref("phyai.models.cosmos3.modeling_cosmos3")
    rot = ref("phyai.layers.rotary_embedding")
    assert torch.equal(mine.compute_mrope_position_ids_text(7, 3)[0], theirs.compute_mrope_position_ids_text(7, 3)[0])
    cases = [dict(fps=None), dict(fps=24.0), dict(fps=10.0), dict(fps=30.0, temporal_compression_factor=1, base_temporal_compression_factor=4,
                                                                   start_frame_offset=1), dict(fps=12.0, enable_fps_modulation=False)]
    for kw in cases:
        a, na = mine.compute_mrope_position_ids_vision(3, 2, 4, 107, **kw)
        b, nb = theirs.compute_mrope_position_ids_vision(3, 2, 4, 107, **kw)
        assert a.dtype == b.dtype and torch.equal(a, b) and na == nb, kw
    for head_dim, sections, theta in ((128, (24, 20, 20), 5e6), (16, (4, 2, 2), 1e4), (64, (16, 8, 8), 1e6)):
        pos = torch.stack([torch.rand(9) * 500, torch.randint(0, 40, (9,)).float(), torch.randint(0, 60, (9,)).float()])
        ours = MRotaryEmbedding(head_dim, sections, theta, interleaved=True)
        cos, sin = rot.compute_qwen3vl_mrope_cos_sin_from_inv_freq(pos[:, None], ours.inv_freq, sections)
        got = ours.cos_sin(pos)
        half = head_dim // 2
        assert torch.allclose(got[:, :half], cos[0, :, :half], atol=1e-6) and torch.allclose(got[:, half:], sin[0, :, :half], atol=1e-6)


def test_pi05_state_bins_and_prompts(ref):
    from phyai_b200.tools import pi05 as mine

    theirs = ref("phyai_utils_tools.models.pi05.ops_pi05")
    g = torch.Generator().manual_seed(0)
    state = torch.cat([torch.rand(4, 9, generator=g) * 2.4 - 1.2, torch.tensor([[-1.0, 1.0, 0.0, -1 + 2 / 256, 1 - 2 / 256, 0.5, -0.5, 2.0, -2.0]])])
    for s in (state, state.bfloat16()):
        assert np.array_equal(mine.discretize_state(s), theirs.discretize_state(s))
    bins = mine.discretize_state(state)
    tasks = ["pick_up the cube", " fold\nthe towel ", "open__drawer", "x", "Wipe The Table"]
    assert mine.build_prompts(tasks, bins) == theirs.build_prompts(tasks, bins)
    assert mine.STATE_NUM_BINS == theirs.STATE_NUM_BINS


def test_cosmos3_prompt_and_bucket_helpers(ref):
    from phyai_b200.tools import cosmos3 as mine

    theirs = ref("phyai_utils_tools.models.cosmos3.steps_cosmos3")
    assert mine.EMBODIMENT_TO_DOMAIN_ID == theirs.EMBODIMENT_TO_DOMAIN_ID
    assert mine.EMBODIMENT_TO_RAW_ACTION_DIM == theirs.EMBODIMENT_TO_RAW_ACTION_DIM
    for h, w in ((720, 1280), (1280, 720), (480, 640), (500, 500), (333, 1000), (1000, 333), (1080, 1920)):
        for tier in ("256", "480", "704", "768", "1080"):
            assert mine.find_closest_target_size(h, w, tier) == theirs.find_closest_target_size(h, w, tier), (h, w, tier)
    for name in ("libero", "LIBERO", " droid_lerobot ", 7):
        assert mine.resolve_domain_id(name) == theirs.resolve_domain_id(name)
    for name in ("pusht", "agibotworld", "robomind-franka-dual"):
        assert mine.resolve_raw_action_dim(name) == theirs.resolve_raw_action_dim(name)
    for prompt, frames, fps, h, w in (("open the drawer", 33, 10.0, 480, 832), ("Stop!", 125, 30.0, 704, 1280), ("wave", 1, 24.0, 100, 150),
                                      ("pour water.", 700, 10.0, 544, 736)):
        for view in ("ego", "wrist", "third_person", "nowhere"):
            kw = dict(view_point=view, num_frames=frames, fps=fps, height=h, width=w)
            assert json.loads(mine.cosmos3_action_json_caption(prompt, **kw)) == json.loads(theirs.cosmos3_action_json_caption(prompt, **kw))
            assert mine.cosmos3_action_json_caption(prompt, **kw) == theirs.cosmos3_action_json_caption(prompt, **kw)
    for prompt in ("A robot arm", "A robot arm.", '{"scene": "lab"}', '{"scene": "lab", "duration": "2s", "fps": 3}', "[1, 2]", "  spaced  "):
        for frames, fps in ((93, 24.0), (1, 24.0), (17, 16.0)):
            for ar in (None, "16,9"):
                kw = dict(fps=fps, num_frames=frames, height=720, width=1280, aspect_ratio=ar)
                assert mine.cosmos3_generation_caption(prompt, **kw) == theirs.cosmos3_generation_caption(prompt, **kw), (prompt, kw)


def test_image_resize_and_normalisation_steps(ref):
    from phyai_b200.tools import processing as mine

    ops, types, steps = (ref(f"phyai_utils_tools.processing.{m}") for m in ("ops.image_ops", "types", "steps.normalize_steps"))
    keys = ref("phyai_utils_tools.processing")
    g = torch.Generator().manual_seed(1)
    for shape, target in (((2, 3, 100, 200), (224, 224)), ((1, 3, 200, 100), (224, 224)), ((1, 3, 37, 53), (64, 48)), ((1, 3, 64, 64), (64, 64))):
        img = torch.rand(*shape, generator=g)
        assert torch.allclose(mine.resize_with_pad(img, *target), ops.resize_with_pad(img, *target), atol=1e-6), (shape, target)
        u8 = (img * 255).to(torch.uint8)
        assert torch.equal(mine.resize_with_pad(u8, *target), ops.resize_with_pad(u8, *target))
    assert torch.equal(mine.normalize_pixels(img), ops.normalize_pixels(img))
    stats = {"observation.state": {"mean": [0.5, -1.0, 2.0], "std": [1.5, 0.5, 2.0], "min": [-1.0, -2.0, 0.0], "max": [2.0, 0.0, 4.0],
                                   "q01": [-0.5, -1.8, 0.2], "q99": [1.5, -0.2, 3.8], "q10": [0.0, -1.5, 1.0], "q90": [1.0, -0.5, 3.0]}}
    x = torch.randn(4, 3, generator=g)
    for mode in ("MEAN_STD", "MIN_MAX", "QUANTILES", "QUANTILE10", "IDENTITY"):
        outs = []
        for ty, st, key in ((mine, mine, mine.STATE), (types, steps, keys.STATE)):
            feats = {"observation.state": ty.PolicyFeature(ty.FeatureType.STATE, (3,))}
            kw = dict(features=feats, norm_map={ty.FeatureType.STATE: ty.NormalizationMode(mode)}, stats=stats)
            y = st.NormalizerStep(**kw)({key: x.clone()})[key]
            outs.append((y, st.UnnormalizerStep(**kw)({key: y.clone()})[key]))
        assert torch.allclose(outs[0][0], outs[1][0], atol=1e-6), mode
        assert torch.allclose(outs[0][1], outs[1][1], atol=1e-6) and torch.allclose(outs[0][1], x, atol=1e-5), mode


class _ChatTokenizer:
    """Bytes + 3 as ids, with the two calls the Cosmos3 processors make on a tokenizer."""

    eos_token_id = 2

    def convert_tokens_to_ids(self, tok):
        return 7

    def apply_chat_template(self, chat, tokenize=True, add_generation_prompt=True):
        text = "".join(f"<{m['role']}>{m['content']}" for m in chat) + "<assistant>"
        return [b + 3 for b in text.encode()]


def test_cosmos3_policy_image_preprocessing(ref):
    from phyai_b200.tools import cosmos3 as mine
    from phyai_b200.tools.processing import IMAGES, PIXEL_VALUES

    theirs = ref("phyai_utils_tools.models.cosmos3.steps_cosmos3")
    rng = np.random.RandomState(0)
    for h, w in ((96, 128), (480, 640), (720, 1280), (300, 200), (1000, 900)):
        img = (rng.rand(h, w, 3) * 255).astype("uint8")
        for th, tw in ((480, 832), (256, 320), (544, 736)):
            assert np.array_equal(mine.resize_and_pad_action_image(img, th, tw), theirs._resize_and_pad_action_image(img, th, tw)), (h, w, th, tw)
        for kw in (dict(height=480, width=832, mode="policy"), dict(height=1, width=1, mode="policy", image_size=480),
                   dict(height=1, width=1, mode="policy", image_size=224)):
            a, b = mine.Cosmos3ImagePreprocessStep(**kw)({IMAGES: img}), theirs.Cosmos3ImagePreprocessStep(**kw)({IMAGES: img})
            assert torch.equal(a[PIXEL_VALUES], b[PIXEL_VALUES]) and a[mine.VIDEO_SHAPE] == b[theirs.VIDEO_SHAPE], (h, w, kw)
            assert (a[mine.META_HEIGHT], a[mine.META_WIDTH]) == (b["meta_height"], b["meta_width"])
    # the other input forms: channel-first tensors in [0, 1] and in [-1, 1], float arrays, several frames
    frames = [torch.rand(3, 64, 96), torch.rand(3, 64, 96) * 2 - 1, rng.rand(64, 96, 3).astype("float32")]
    kw = dict(height=48, width=80, mode="inverse_dynamics")
    a, b = mine.Cosmos3ImagePreprocessStep(**kw)({IMAGES: frames}), theirs.Cosmos3ImagePreprocessStep(**kw)({IMAGES: frames})
    assert torch.equal(a[PIXEL_VALUES], b[PIXEL_VALUES]) and a[mine.VIDEO_SHAPE] == b[theirs.VIDEO_SHAPE] == (3, 48, 80)
    assert mine.Cosmos3ImagePreprocessStep(**kw).get_config() == theirs.Cosmos3ImagePreprocessStep(**kw).get_config()


def test_cosmos3_policy_processor_end_to_end(ref, tmp_path, monkeypatch):
    from phyai_b200.tools import cosmos3 as mine

    theirs = ref("phyai_utils_tools.models.cosmos3.processor_cosmos3")
    monkeypatch.setattr(theirs, "get_tokenizer", lambda name: _ChatTokenizer())      # no tokenizer files offline
    stats = tmp_path / "stats.json"
    stats.write_text(json.dumps({"global": {"mean": [0.1] * 10, "std": [2.0] * 10, "min": [-1.0] * 10, "max": [3.0] * 10, "q01": [-0.5] * 10,
                                            "q99": [2.5] * 10}, "global_raw": {"q01": [-3.0] * 10, "q99": [5.0] * 10}}))
    rng = np.random.RandomState(1)
    img = (rng.rand(240, 320, 3) * 255).astype("uint8")
    act = rng.rand(5, 10).astype("float32")
    cases = [dict(mode="policy", prompt_format="plain", image_size=480), dict(mode="policy", prompt_format="json", image_size=480, view_point="wrist_view"),
             dict(mode="forward_dynamics", prompt_format="plain", append_metadata=False), dict(mode="inverse_dynamics", prompt_format="json", view_point="none"),
             dict(mode="policy", negative_prompt="bad video", fps=10.0, action_chunk_size=32, cond_frame_indexes=(0, 1))]
    for kw in cases:
        common = dict(domain_name="droid_lerobot", **kw)
        a = mine.Cosmos3PolicyProcessor(tokenizer=_ChatTokenizer(), **common)
        b = theirs.Cosmos3PolicyProcessor(tokenizer_name_or_path="unused", **common)
        raw = {"images": img, "task": "put the cup on the plate", "cond_action": act}
        x, y = a.preprocess(dict(raw)), b.preprocess(dict(raw))
        for f in ("pixel_values", "text_ids", "text_mask", "neg_text_ids", "neg_text_mask"):
            assert torch.equal(getattr(x, f), getattr(y, f)), (kw, f)
        assert (x.cond_action is None) == (y.cond_action is None) and (x.cond_action is None or torch.equal(x.cond_action, y.cond_action))
        for f in ("domain_id", "mode", "action_chunk", "raw_action_dim", "video_shape", "cond_frame_indexes"):
            assert getattr(x, f) == getattr(y, f), (kw, f)
    out = {"action": torch.from_numpy(rng.rand(1, 16, 64).astype("float32")) * 2 - 1, "video": torch.zeros(2), "pixels": torch.ones(2)}
    for norm in ("meanstd", "minmax", "quantile", "quantile_rot"):
        common = dict(domain_name="droid_lerobot", action_stats_path=str(stats), action_normalization=norm)
        a = mine.Cosmos3PolicyProcessor(tokenizer=_ChatTokenizer(), **common).postprocess(out)
        b = theirs.Cosmos3PolicyProcessor(tokenizer_name_or_path="unused", **common).postprocess(out)
        assert set(a) == set(b) and torch.allclose(a["action"], b["action"], atol=1e-6) and a["action"].shape == (1, 16, 10), norm
    a = mine.Cosmos3PolicyProcessor(tokenizer=_ChatTokenizer(), domain_name="pusht").postprocess(out["action"])
    b = theirs.Cosmos3PolicyProcessor(tokenizer_name_or_path="unused", domain_name="pusht").postprocess(out["action"])
    assert torch.equal(a["action"], b["action"]) and a["action"].shape == (1, 16, 2)


def test_cosmos3_generation_tokenisation(ref, monkeypatch):
    from phyai_b200.tools import cosmos3 as mine

    theirs = ref("phyai_utils_tools.models.cosmos3.processor_cosmos3")
    monkeypatch.setattr(theirs, "get_tokenizer", lambda name: _ChatTokenizer())
    for kw in (dict(), dict(use_system_prompt=True, fps=24.0, num_frames=93, height=720, width=1280),
               dict(fps=16.0, num_frames=1, height=480, width=832, aspect_ratio="16,9"), dict(fps=24.0, num_frames=93, height=720, width=1280, append_metadata=False),
               dict(negative_prompt="ugly")):
        a, b = mine.Cosmos3Processor(tokenizer=_ChatTokenizer(), **kw), theirs.Cosmos3Processor("unused", **kw)
        for prompt in ("A robot arm stacks cups", '{"scene": "lab"}'):
            for neg in (None, "", "blurry"):
                if neg is None and "negative_prompt" not in kw:
                    continue          # the default negative prompt is a data file of the upstream release, not part of this package
                (p1, n1), (p2, n2) = a.tokenize_pair(prompt, neg), b.tokenize_pair(prompt, neg)
                assert torch.equal(p1.text_ids, p2.text_ids) and torch.equal(n1.text_ids, n2.text_ids) and torch.equal(p1.text_mask, p2.text_mask)
    shipped = REF / "phyai_utils_tools" / "models" / "cosmos3" / "neg_prompts.json"
    if shipped.is_file():             # given the release's file, the default negative prompt is the reference's byte for byte
        assert mine.cosmos3_default_negative_prompt(shipped) == ref("phyai_utils_tools.models.cosmos3.steps_cosmos3").cosmos3_default_negative_prompt()


def _same_inputs(x, y, fields):
    for f in fields:
        a, b = getattr(x, f), getattr(y, f)
        assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b), f


@pytest.mark.parametrize("model", ["pi05", "pi0"])
def test_policy_processors_and_their_saved_files(ref, tmp_path, model):
    """Same arguments, same sample: the same request tensors and the same actions; and a processor saved by either
    package loads in the other and behaves the same (the files are lerobot's format)."""
    from phyai_b200.tools import pi0 as my_pi0
    from phyai_b200.tools import pi05 as my_pi05
    from phyai_b200.tools.tokenizer import ByteTokenizer

    if model == "pi05":
        mine, theirs = my_pi05.PI05Processor, ref("phyai_utils_tools.models.pi05.processor_pi05").PI05Processor
        # the reference un-normalises before it cuts the action, so its statistics span the model's whole action width
        stats = {"observation.state": {"q01": [-1.0, 0.0, -2.0], "q99": [1.0, 4.0, 2.0]},
                 "action": {"q01": [-1.0] * 32, "q99": [3.0, 2.0, 1.0, 0.5] * 8}}
        fields = ("pixel_values", "input_ids", "lang_lens")
    else:
        mine, theirs = my_pi0.PI0Processor, ref("phyai_utils_tools.models.pi0.processor_pi0").PI0Processor
        stats = {"observation.state": {"mean": [0.5, 1.0, -1.0], "std": [2.0, 0.5, 1.5]}, "action": {"mean": [0.1] * 4, "std": [2.0, 1.0, 0.5, 0.25]}}
        fields = ("pixel_values", "input_ids", "lang_lens", "state")
    tok = ByteTokenizer()
    g = torch.Generator().manual_seed(0)
    sample = {"images": [torch.rand(2, 3, 40, 64, generator=g), torch.rand(2, 3, 64, 40, generator=g)],
              "state": torch.rand(2, 3, generator=g) * 2 - 1, "task": ["Pick_up the cube", "fold the\ntowel"]}
    action = torch.rand(2, 6, 32, generator=g) * 2 - 1
    for kw in (dict(dataset_stats=stats, action_dim=4, normalize_pixels=True), dict(dataset_stats=None, action_dim=None, normalize_pixels=False),
               dict(dataset_stats=stats, action_dim=7 if model == "pi05" else 4, image_pad_value=-1.0)):
        common = dict(tokenizer=tok, image_size=32, num_images=2, tokenizer_max_length=96, params_dtype=torch.float32, **kw)
        a, b = mine(**common), theirs(**common)
        _same_inputs(a.preprocess({k: (list(v) if isinstance(v, list) else v) for k, v in sample.items()}),
                     b.preprocess({k: (list(v) if isinstance(v, list) else v) for k, v in sample.items()}), fields)
        ya, yb = a.postprocess(action.clone()), b.postprocess(action.clone())
        assert ya.shape == yb.shape and ya.dtype == yb.dtype and torch.allclose(ya, yb, atol=1e-6), kw
    # saved by one, loaded by the other
    common = dict(tokenizer=tok, image_size=32, num_images=2, tokenizer_max_length=96, params_dtype=torch.float32, dataset_stats=stats, action_dim=4)
    a, b = mine(**common), theirs(**common)
    a.save_pretrained(tmp_path / "mine")
    b.save_pretrained(tmp_path / "theirs")
    load = dict(tokenizer=tok, image_size=32, num_images=2, action_dim=4, params_dtype=torch.float32)
    if model == "pi0":
        load["normalize_pixels"] = True
    want_in, want_out = b.preprocess(dict(sample)), b.postprocess(action.clone())
    for loader, folder in ((mine, "theirs"), (theirs, "mine"), (mine, "mine")):
        p = loader.from_pretrained(tmp_path / folder, **load)
        _same_inputs(p.preprocess(dict(sample)), want_in, fields)
        assert torch.allclose(p.postprocess(action.clone()), want_out, atol=1e-6), (loader.__module__, folder)
    for name in ("policy_preprocessor.json", "policy_postprocessor.json"):
        ja, jb = (json.loads((tmp_path / d / name).read_text()) for d in ("mine", "theirs"))
        assert [s["registry_name"] for s in ja["steps"]] == [s["registry_name"] for s in jb["steps"]], name


def test_default_configurations(ref):
    """Every field of the default model configurations (nested ones included) has the reference's value, so a checkpoint's
    ``config.json`` that leaves a field out means the same model in both packages."""
    import dataclasses

    def flat(x, pre=""):
        out = {}
        for f in dataclasses.fields(x):
            v = getattr(x, f.name)
            if dataclasses.is_dataclass(v):
                out.update(flat(v, pre + f.name + "."))
            else:
                out[pre + f.name] = list(v) if isinstance(v, (tuple, list)) else v
        return out

    for mod, cls in (("models.pi05.configuration_pi05", "PI05Config"), ("models.pi0.configuration_pi0", "PI0Config"),
                     ("models.cosmos3.configuration_cosmos3", "Cosmos3Config"), ("models.cosmos3.configuration_cosmos3", "Cosmos3WanVAEConfig"),
                     ("models.cosmos3.configuration_cosmos3", "Cosmos3AVAESoundConfig")):
        mine = flat(getattr(importlib.import_module("phyai_b200." + mod), cls)())
        theirs = flat(getattr(ref("phyai." + mod), cls)())
        theirs.pop("expert.adarms_cond_dim", None) if cls == "PI0Config" else None      # Pi0 has no time-conditioned norm: the width is unused
        mine.pop("expert.adarms_cond_dim", None) if cls == "PI0Config" else None
        assert mine == theirs, (cls, {k: (mine.get(k), theirs.get(k)) for k in set(mine) | set(theirs) if mine.get(k) != theirs.get(k)})


@pytest.fixture()
def ref_single_rank(ref):
    """The reference's process-level state for building its models on CPU: engine configuration on the CPU in fp32 and a
    single-rank mesh under its default name (a stand-in for the torch device mesh, as its own unit tests use)."""
    from unittest.mock import MagicMock

    ec, mesh, state = ref("phyai.engine_config"), ref("phyai.parallel.mesh"), ref("phyai.parallel.state")
    saved_cfg, saved_meshes = ec.get_engine_config(), dict(state._meshes)
    ec.set_engine_config(saved_cfg.replace(device=ec.DeviceConfig(target="cpu", params_dtype=torch.float32)))
    tm = MagicMock()
    tm.mesh_dim_names = ("dp", "cfg", "ep", "sp", "cp", "tp")
    tm.size.side_effect = lambda axis: 1
    tm.get_local_rank.side_effect = lambda axis: 0
    tm.get_group.side_effect = lambda axis: MagicMock(name=f"pg-{axis}")
    state.register_mesh(mesh.Mesh(tm, name="model"))
    try:
        yield ref
    finally:
        ec.set_engine_config(saved_cfg)
        state._meshes.clear()
        state._meshes.update(saved_meshes)


def _mirror_config(cfg, module):
    """The reference's configuration object with the field values of this package's (class names and fields coincide)."""
    import dataclasses

    if dataclasses.is_dataclass(cfg):
        return getattr(module, type(cfg).__name__)(**{f.name: _mirror_config(getattr(cfg, f.name), module) for f in dataclasses.fields(cfg)})
    return cfg


@pytest.mark.parametrize("what", ["cosmos3", "cosmos3_action", "cosmos3_sound", "pi05", "pi0"])
def test_checkpoints_written_from_this_package_load_strictly_into_the_reference(ref_single_rank, tmp_path, what):
    """One tensor per checkpoint key this package's model expects (fused parameters: one per leg), written as a
    checkpoint, is loaded by the reference's loader into the reference's model with ``strict=True``: the two models
    expect the same key names and shapes. Parameters that exist under one name in both hold the same values afterwards."""
    from phyai_b200 import parallel as P
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.weights import synthetic_state_dict, write_checkpoint

    ref = ref_single_rank
    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    P.init((1,), ("tp",), device="cpu")
    try:
        if what.startswith("cosmos3"):
            from phyai_b200.models.cosmos3 import Cosmos3Transformer, tiny_cosmos3_config
            from phyai_b200.models.cosmos3.transformer_cosmos3 import cosmos3_inverse_remap

            rm = ref("phyai.models.cosmos3.modeling_cosmos3")
            cfg = tiny_cosmos3_config(action_gen=what.endswith("action"), sound_gen=what.endswith("sound"))
            mine = Cosmos3Transformer(cfg, params_dtype=torch.float32, device="cpu")
            theirs = rm.Cosmos3Transformer(_mirror_config(cfg, rm), params_dtype=torch.float32, device="cpu")
            state = {cosmos3_inverse_remap(k): v for k, v in synthetic_state_dict(mine, seed=1, std=0.05).items()}
            remap = rm.cosmos3_weight_remap
        elif what == "pi05":
            from phyai_b200.models.pi05.configuration_pi05 import tiny_pi05_config
            from phyai_b200.models.pi05.modeling_pi05 import PI05Model

            cfg = tiny_pi05_config()
            mine = PI05Model(cfg)
            # building the reference's model touches no GPU; its paged attention layers only accept this backend name
            theirs = ref("phyai.models.pi05.modeling_pi05").PI05Model(_mirror_config(cfg, ref("phyai.models.pi05.configuration_pi05")),
                                                                      attn_backend="flashinfer", norm_backend="flashinfer", device="cpu")
            ref("phyai.engine")          # the plugin modules import one another through it
            state, remap = synthetic_state_dict(mine, seed=1, std=0.05), ref("phyai.models.pi05.main_pi05")._compose_remap(None)
        else:
            from phyai_b200.models.pi0.configuration_pi0 import tiny_pi0_config
            from phyai_b200.models.pi0.main_pi0 import compose_remap
            from phyai_b200.models.pi0.modeling_pi0 import PI0Model

            cfg = tiny_pi0_config()
            mine = PI0Model(cfg)
            theirs = ref("phyai.models.pi0.modeling_pi0").PI0Model(_mirror_config(cfg, ref("phyai.models.pi0.configuration_pi0")),
                                                                   attn_backend="flashinfer", norm_backend="flashinfer", device="cpu")
            ref("phyai.engine")
            state, remap = synthetic_state_dict(mine, seed=1, std=0.05), ref("phyai.models.pi0.main_pi0")._compose_remap(None)
        gs = torch.Generator().manual_seed(2)
        state = {k: (torch.randn(v.shape, generator=gs) * 0.1).to(v.dtype) if float(v.float().abs().sum()) == 0 or bool((v == 1).all()) else v
                 for k, v in state.items()}          # identity norms and zero tables would hide a mix-up: every tensor random
        write_checkpoint(tmp_path, state, None)
        report = ref("phyai.weights.loader").load_pretrained(theirs, tmp_path, remap=remap, strict=True)
        assert not report.missing and not report.unexpected, (report.missing[:5], report.unexpected[:5])
        theirs_named = dict(theirs.named_parameters())
        from phyai_b200.weights import load_pretrained

        if what.startswith("cosmos3"):
            from phyai_b200.models.cosmos3.transformer_cosmos3 import cosmos3_weight_remap

            load_pretrained(mine, tmp_path, remap=cosmos3_weight_remap, strict=True)
        else:
            load_pretrained(mine, tmp_path, strict=True)
        shared = [(n, p) for n, p in mine.named_parameters() if n in theirs_named and theirs_named[n].shape == p.shape]
        assert len(shared) >= 5
        for n, p in shared:
            a, b = p.data.float(), theirs_named[n].data.float()
            if "gate_up" in n and not torch.equal(a, b):
                # this package keeps gate and up rows interleaved (the gated epilogue reads them as neighbours), the
                # reference one block after the other
                half = b.shape[0] // 2
                assert torch.equal(a[0::2], b[:half]) and torch.equal(a[1::2], b[half:]), n
            else:
                assert torch.equal(a, b), n
    finally:
        P.shutdown()


def test_video_vae_and_sound_decoder_numerics(ref_single_rank, tmp_path):
    """The convolutional parts run on the CPU in both packages: one checkpoint (this package's key index, every tensor
    random), the reference's loader and model on one side, this package's on the other; decoded pixels, encoded latents and
    the decoded waveform agree to fp32 rounding (the reference walks the clip in chunks of frames with a feature cache,
    this package in one pass or a stream)."""
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.models.cosmos3 import Cosmos3AVAESoundConfig, Cosmos3WanVAEConfig
    from phyai_b200.models.cosmos3.avae_sound import Cosmos3AVAESoundDecoder, cosmos3_avae_weight_remap
    from phyai_b200.models.cosmos3.vae_wan import Cosmos3WanVAE, cosmos3_vae_weight_remap
    from phyai_b200.weights import load_pretrained, synthetic_state_dict, write_checkpoint

    ref = ref_single_rank
    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    rcfg, rvae, ravae, rload = (ref(m) for m in ("phyai.models.cosmos3.configuration_cosmos3", "phyai.models.cosmos3.vae_wan",
                                                 "phyai.models.cosmos3.avae_sound", "phyai.weights.loader"))
    gs = torch.Generator().manual_seed(0)

    def randomised(model):
        st = synthetic_state_dict(model, seed=3, std=0.05)
        return {k: (torch.randn(v.shape, generator=gs) * (0.3 if v.dim() > 1 else 0.1) + (1.0 if v.dim() == 1 and "gamma" in k else 0.0)).to(v.dtype)
                for k, v in st.items()}

    # ---- video VAE
    cfg = Cosmos3WanVAEConfig(z_dim=4, decoder_base_dim=8, base_dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1,
                              latents_mean=tuple(0.1 * i for i in range(4)), latents_std=tuple(1.0 + 0.1 * i for i in range(4)))
    mine = Cosmos3WanVAE(cfg, device="cpu", dtype=torch.float32).eval()
    d = tmp_path / "vae"
    write_checkpoint(d, randomised(mine), None)
    load_pretrained(mine, d, remap=cosmos3_vae_weight_remap, strict=True)
    theirs = rvae.Cosmos3WanVAE(_mirror_config(cfg, rcfg)).eval()
    rep = rload.load_pretrained(theirs, d, remap=rvae.cosmos3_vae_weight_remap, strict=True)
    assert not rep.missing and not rep.unexpected
    lat = torch.randn(1, 4, 3, 4, 6, generator=gs)
    with torch.no_grad():
        a, b = mine.decode(lat), theirs.decode(lat)
        assert a.shape == b.shape == (1, 3, 9, 64, 96)
        assert torch.allclose(a, b, atol=2e-4, rtol=1e-4), (a - b).abs().max()
        assert torch.allclose(mine.decode(lat, frames_per_chunk=1), b, atol=2e-4, rtol=1e-4)
        pix = torch.rand(1, 3, 5, 32, 48, generator=gs) * 2 - 1
        ea, eb = mine.encode(pix), theirs.encode(pix)
        assert ea.shape == eb.shape == (1, 4, 2, 2, 3) and torch.allclose(ea, eb, atol=2e-4, rtol=1e-4), (ea - eb).abs().max()

    # ---- sound decoder
    acfg = Cosmos3AVAESoundConfig(latent_ch=8, dec_dim=16, dec_c_mults=(1, 2, 4), dec_strides=(2, 4, 5))
    mine_a = Cosmos3AVAESoundDecoder(acfg, device="cpu", dtype=torch.float32).eval()
    d = tmp_path / "avae"
    # this package also accepts the newer spelling of weight-normalised convolutions (parametrizations.weight.original0 / 1);
    # a checkpoint carries one spelling, here the one the reference knows (weight_g / weight_v)
    write_checkpoint(d, {k: v for k, v in randomised(mine_a).items() if "parametrizations" not in k}, None)
    load_pretrained(mine_a, d, remap=cosmos3_avae_weight_remap, strict=True)
    theirs_a = ravae.Cosmos3AVAESoundDecoder(_mirror_config(acfg, rcfg)).eval()
    rep = rload.load_pretrained(theirs_a, d, remap=ravae.cosmos3_avae_weight_remap, strict=True)
    assert not rep.missing and not rep.unexpected
    z = torch.randn(1, 8, 7, generator=gs)
    with torch.no_grad():
        wa, wb = mine_a.decode(z), theirs_a.decode(z)
    assert wa.shape == wb.shape and wa.shape[-1] == 7 * 40 and torch.allclose(wa, wb, atol=2e-4, rtol=1e-4), (wa - wb).abs().max()


@pytest.mark.parametrize("tp,rank", [(2, 1), (4, 2), (8, 5)])
def test_tensor_parallel_shards_of_one_checkpoint(ref, tmp_path, tp, rank):
    """The same full-size checkpoint tensors loaded by both packages into their parallel layers on rank ``rank`` of ``tp``
    (stand-in meshes, no process group): column / row shards, fused q | k | v with fewer KV heads than ranks (replicated
    KV heads), fused gate / up, vocabulary shards with padding rows."""
    import torch.nn as nn
    from unittest.mock import MagicMock

    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.layers import linear as L
    from phyai_b200.layers.vocab_embedding import VocabParallelEmbedding
    from phyai_b200.parallel.mesh import Mesh
    from phyai_b200.weights import load_pretrained, write_checkpoint

    ec, rmesh, rstate = ref("phyai.engine_config"), ref("phyai.parallel.mesh"), ref("phyai.parallel.state")
    RL, RV, rload = ref("phyai.layers.linear"), ref("phyai.layers.vocab_embedding"), ref("phyai.weights.loader")
    saved_cfg, saved_meshes = ec.get_engine_config(), dict(rstate._meshes)
    ec.set_engine_config(saved_cfg.replace(device=ec.DeviceConfig(target="cpu", params_dtype=torch.float32)))
    tm = MagicMock()
    tm.mesh_dim_names = ("tp",)
    tm.size.side_effect = lambda axis: tp
    tm.get_local_rank.side_effect = lambda axis: rank
    tm.get_group.side_effect = lambda axis: MagicMock(name=f"pg-{axis}")
    rstate.register_mesh(rmesh.Mesh(tm, name="model"))
    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    my_mesh = Mesh((tp,), ("tp",), rank=rank, build_groups=False)
    try:
        H, D, heads, kv_heads, I, V = 64, 8, 16, 2, 48 * tp // 2, 100
        kw = dict(bias=True, params_dtype=torch.float32)

        class Mine(nn.Module):
            def __init__(self):
                super().__init__()
                self.col = L.ColumnParallelLinear(H, 32 * tp, mesh=my_mesh, prefix="col", **kw)
                self.row = L.RowParallelLinear(32 * tp, H, mesh=my_mesh, prefix="row", **kw)
                self.qkv = L.QKVParallelLinear(H, D, heads, kv_heads, mesh=my_mesh, prefix="attn.qkv_proj", hf_legs=("q_proj", "k_proj", "v_proj"), **kw)
                self.gu = L.MergedColumnParallelLinear(H, [I, I], mesh=my_mesh, prefix="mlp.gate_up_proj", hf_legs=("gate_proj", "up_proj"), **kw)
                self.emb = VocabParallelEmbedding(V, H, params_dtype=torch.float32, mesh=my_mesh, device="cpu", prefix="emb")

        class Theirs(nn.Module):
            def __init__(self):
                super().__init__()
                self.col = RL.ColumnParallelLinear(H, 32 * tp, prefix="col", **kw)
                self.row = RL.RowParallelLinear(32 * tp, H, prefix="row", **kw)
                self.qkv = RL.QKVParallelLinear(H, D, heads, kv_heads, prefix="attn.qkv_proj", hf_legs={"q": "q_proj", "k": "k_proj", "v": "v_proj"}, **kw)
                self.gu = RL.MergedColumnParallelLinear(H, [I, I], prefix="mlp.gate_up_proj", hf_legs=("gate_proj", "up_proj"), **kw)
                self.emb = RV.VocabParallelEmbedding(V, H, params_dtype=torch.float32, device="cpu", prefix="emb")

        mine, theirs = Mine(), Theirs()
        g = torch.Generator().manual_seed(tp * 10 + rank)
        r = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
        ck = {"col.weight": r(32 * tp, H), "col.bias": r(32 * tp), "row.weight": r(H, 32 * tp), "row.bias": r(H),
              "attn.q_proj.weight": r(heads * D, H), "attn.k_proj.weight": r(kv_heads * D, H), "attn.v_proj.weight": r(kv_heads * D, H),
              "attn.q_proj.bias": r(heads * D), "attn.k_proj.bias": r(kv_heads * D), "attn.v_proj.bias": r(kv_heads * D),
              "mlp.gate_proj.weight": r(I, H), "mlp.up_proj.weight": r(I, H), "mlp.gate_proj.bias": r(I), "mlp.up_proj.bias": r(I),
              "emb.weight": r(V, H)}
        write_checkpoint(tmp_path, ck, None)
        rep_a = load_pretrained(mine, tmp_path, strict=True)
        rep_b = rload.load_pretrained(theirs, tmp_path, strict=True)
        assert not rep_a.missing and not rep_b.missing and not rep_a.unexpected and not rep_b.unexpected
        for name in ("col", "row", "qkv", "emb"):
            for pn, p in getattr(mine, name).named_parameters():
                q = dict(getattr(theirs, name).named_parameters())[pn]
                assert p.shape == q.shape and torch.equal(p.data, q.data), (name, pn)
        # gate / up: both hold this rank's gate block and up block; this package may interleave their rows
        for pn, p in mine.gu.named_parameters():
            q = dict(theirs.gu.named_parameters())[pn]
            assert p.shape == q.shape
            half = q.shape[0] // 2
            same = torch.equal(p.data, q.data) or (torch.equal(p.data[0::2], q.data[:half]) and torch.equal(p.data[1::2], q.data[half:]))
            assert same, pn
        # what the shards must be, said directly
        per = 32
        assert torch.equal(mine.col.weight.data, ck["col.weight"][rank * per:(rank + 1) * per]) and torch.equal(mine.row.weight.data, ck["row.weight"][:, rank * per:(rank + 1) * per])
        hq = heads // tp
        assert torch.equal(mine.qkv.weight.data[: hq * D], ck["attn.q_proj.weight"][rank * hq * D:(rank + 1) * hq * D])
        kv_of_rank = rank * kv_heads // tp if tp > kv_heads else None
        if kv_of_rank is not None:      # more ranks than KV heads: each rank holds one whole KV head, shared by tp / kv_heads ranks
            assert torch.equal(mine.qkv.weight.data[hq * D: hq * D + D], ck["attn.k_proj.weight"][kv_of_rank * D:(kv_of_rank + 1) * D])
    finally:
        ec.set_engine_config(saved_cfg)
        rstate._meshes.clear()
        rstate._meshes.update(saved_meshes)


def test_quantisation_plans_from_checkpoint_configs(ref, tmp_path):
    """The three checkpoint dialects (HF fp8, compressed-tensors, ModelOpt) read from a folder by both packages: the same
    modules are quantised and the same are left alone, with the same weight format (element type, granularity, block
    shape). Entries are exact module names, last path components, class targets and ``re:`` patterns, which both packages
    read the same way (this package additionally understands globs and path components inside a dotted name)."""
    from phyai_b200.layers.linear import LinearBase as MyLinear
    from phyai_b200.layers.quant import load_quant_plan

    theirs_load = ref("phyai.layers.quant.active").load_quant_plan
    TheirLinear = ref("phyai.layers.linear").LinearBase
    cases = {
        "hf_block": ("config.json", {"quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128], "modules_to_not_convert": ["lm_head", "fc1"]}}),
        "hf_plain": ("config.json", {"quantization_config": {"quant_method": "fp8", "ignored_layers": ["model.layers.3.mlp.down_proj"]}}),
        "ct_channel": ("config.json", {"quantization_config": {"quant_method": "compressed-tensors", "ignore": ["lm_head", "re:.*vision.*"], "config_groups": {"g": {
            "targets": ["Linear"], "weights": {"num_bits": 8, "type": "float", "strategy": "channel"},
            "input_activations": {"num_bits": 8, "type": "float", "strategy": "token", "dynamic": True}}}}}),
        "ct_regex_from_start": ("config.json", {"compression_config": {"quant_method": "compressed-tensors", "config_groups": {"g": {
            "targets": ["re:model\\\\.layers\\\\.\\\\d+\\\\.mlp", "re:mlp"], "weights": {"num_bits": 8, "type": "float", "strategy": "tensor"}}}}}),
        "ct_block_named": ("config.json", {"quantization_config": {"quant_method": "compressed-tensors", "config_groups": {"g": {
            "targets": ["model.layers.0.self_attn.q_proj", "down_proj"], "weights": {"num_bits": 8, "type": "float", "strategy": "block", "block_structure": [128, 128]}}}}}),
        "modelopt_fp4": ("hf_quant_config.json", {"quantization": {"quant_algo": "NVFP4", "exclude_modules": ["lm_head", "vision.proj"]}}),
        "modelopt_inline": ("config.json", {"quantization_config": {"quant_method": "modelopt", "quant_algo": "NVFP4", "ignore": ["lm_head"]}}),
    }
    names = ["model.layers.0.self_attn.q_proj", "model.layers.3.mlp.down_proj", "lm_head", "model.vision_tower.blocks.0.fc1", "vision.proj", "mlp.up_proj"]

    def weight_format(scheme):
        if scheme is None:
            return None
        w = scheme.weight
        gran = w.granularity.value if hasattr(w.granularity, "value") else str(w.granularity)
        return (w.dtype.value, "block" if w.dtype.value == "nvfp4" else gran.lower(), tuple(w.block_shape) if gran.lower() == "block" and w.block_shape else None)

    for tag, (fname, blob) in cases.items():
        d = tmp_path / tag
        d.mkdir()
        (d / "config.json").write_text(json.dumps({"hidden_size": 8, **(blob if fname == "config.json" else {})}))
        if fname != "config.json":
            (d / fname).write_text(json.dumps(blob))
        pa, pb = load_quant_plan(d), theirs_load(d)
        assert pa is not None and pb is not None, tag
        for n in names:
            a, b = weight_format(pa.resolve(n, MyLinear)), weight_format(pb.resolve(n, TheirLinear))
            if a is not None and b is not None and a[0] == b[0] == "fp8_e4m3" and {a[1], b[1]} == {"per_tensor", "per_channel"}:
                continue      # one scale per tensor in the file; both packages fan it out per channel after loading
            assert a == b, (tag, n, a, b)


def test_prefix_cache_encodings_and_behaviour(ref):
    """The prompt encodings byte for byte, and one scripted life of a prefix cache (inserts that share prefixes, matches
    that split edges, a full device tier under each eviction policy) against the reference's native cache: the same
    match lengths, unit counts and inserted / freed numbers at every step."""
    import hashlib
    import random

    from phyai_b200.cache import radix_cache as mine

    theirs, native = ref("phyai.cache.radix_cache"), ref("phyai_ext.radix_cache")
    enc = ref("phyai.cache.radix_cache.encoding")
    rng = random.Random(0)
    ids = [rng.randrange(0, 2 ** 31 - 1) for _ in range(37)]
    assert mine.encode_text_atoms_int32(ids) == enc.encode_text_atoms_int32(ids)
    assert mine.encode_eagle_bigram_atoms(ids) == enc.encode_eagle_bigram_atoms(ids)
    hashes = [rng.randrange(0, 2 ** 64) for _ in range(9)]
    assert mine.encode_chunk_hash_atoms_u64(hashes) == enc.encode_chunk_hash_atoms_u64(hashes)
    digest = hashlib.sha256(b"image").digest()
    assert mine.encode_image_hash_atom_sha256(digest) == enc.encode_image_hash_atom_sha256(digest)
    segs = [(5, 3), (20, 4)]
    a = mine.encode_prompt_to_atoms(ids, [mine.ImageSegment(11 + i, 22 + i, p, n) for i, (p, n) in enumerate(segs)])
    b = enc.encode_prompt_to_atoms(ids, [enc.ImageSegment(11 + i, 22 + i, p, n) for i, (p, n) in enumerate(segs)])
    assert a == b
    for page in (8, 16, 64):
        assert mine.page_align(a, page) == enc.page_align(b, page)

    def life(mod, cache_cls, tier):
        """Inserts that share prefixes and matches that split edges, in a tier large enough that nothing is evicted."""
        c = cache_cls(atom_bytes=4, atoms_per_unit=2, device_total_units=64)
        log = [("page", c.page_bytes, c.total(tier), c.available(tier))]
        r = random.Random(7)
        seqs = [[r.randrange(0, 50) for _ in range(r.choice((4, 6, 8, 10)))] for _ in range(6)]
        seqs += [seqs[0][:4] + [91, 92, 93, 94], seqs[1][:2] + [81, 82], seqs[0][:4] + [91, 92, 71, 72], seqs[0][:3]]
        for s_ in seqs:
            atoms, _ = mod.page_align(mod.encode_text_atoms_int32(s_), c.page_bytes)
            log.append(("match", c.match(atoms).matched_atoms[0]))
            need = len(atoms) // c.page_bytes
            if need:
                _, inserted, freed = c.insert(tier, atoms, c.allocate(tier, need))
                log.append(("insert", inserted, freed, c.active(tier), c.available(tier)))
            log.append(("rematch", c.match(atoms).matched_atoms[0]))
            c.advance_step(1)
        return log

    assert life(mine, mine.PrefixCache, mine.Tier.DEVICE) == life(enc, native.PrefixCache, native.Tier.DEVICE)

    def eviction(mod, cache_cls, tier, policy):
        """Three one-page prefixes with distinct recency and hit counts fill the tier; room for two pages is asked for."""
        c = cache_cls(atom_bytes=4, atoms_per_unit=1, device_total_units=7, eviction_policy=policy, slru_threshold=2)
        tok = mod.encode_text_atoms_int32
        for ids in ([1, 2], [3, 4], [5, 6]):
            c.insert(tier, tok(ids), c.allocate(tier, 2))
            c.advance_step(1)
        c.match(tok([1, 2]))
        c.advance_step(1)
        c.match(tok([1, 2]))
        c.advance_step(1)
        c.match(tok([5, 6]))
        c.advance_step(1)
        c.ensure_capacity(tier, 2)
        return [c.match(tok(ids)).matched_atoms[0] for ids in ([1, 2], [3, 4], [5, 6])], c.available(tier)

    for policy in ("lru", "lfu", "slru"):
        got = eviction(mine, mine.PrefixCache, mine.Tier.DEVICE, policy)
        want = eviction(enc, native.PrefixCache, native.Tier.DEVICE, policy)
        assert got == want == ([2, 0, 2], 2), (policy, got, want)       # the prefix that is neither recent nor hot goes


def test_environment_catalogue_and_engine_config_fields(ref, monkeypatch):
    """Every ``PHYAI_*`` variable and every engine configuration field of the reference exists here with the same default
    (backend names differ: this package's kernels are its own), and the same environment gives the same configuration."""
    import dataclasses

    from phyai_b200 import engine_config as mine_ec
    from phyai_b200 import env as mine_env

    their_env, their_ec = ref("phyai.env"), ref("phyai.engine_config")
    names = lambda mod: {k: v for k, v in vars(mod.envs).items() if k.startswith("PHYAI_")}  # noqa: E731
    a, b = names(mine_env), names(their_env)
    assert set(b) <= set(a), sorted(set(b) - set(a))
    for k in b:
        assert getattr(a[k], "default", None) == getattr(b[k], "default", None), k
    for cls in ("BackendConfig", "DeviceConfig", "ParallelConfig", "RuntimeConfig"):
        fa = {f.name: f.default for f in dataclasses.fields(getattr(mine_ec, cls))}
        fb = {f.name: f.default for f in dataclasses.fields(getattr(their_ec, cls))}
        assert set(fb) <= set(fa), (cls, sorted(set(fb) - set(fa)))
        diff = {k for k in fb if fa[k] != fb[k] and not callable(fa[k])}
        assert diff <= ({"attn", "norm"} if cls == "BackendConfig" else set()), (cls, diff)
    for k, v in {"PHYAI_DEVICE": "cpu", "PHYAI_PARAMS_DTYPE": "float16", "PHYAI_FORCE_LINEAR_KERNEL": "torch",
                 "PHYAI_DEBUG_TENSOR_DUMP_DIR": "/tmp/x", "PHYAI_DEBUG_TENSOR_DUMP_FILTER": "a.*,b$", "PHYAI_FLASHINFER_WORKSPACE_BYTES": "1048576"}.items():
        monkeypatch.setenv(k, v)

    def flat(x, pre=""):
        out = {}
        for f in dataclasses.fields(x):
            v = getattr(x, f.name)
            out.update(flat(v, pre + f.name + ".")) if dataclasses.is_dataclass(v) else out.update({pre + f.name: str(v)})
        return out

    fa, fb = flat(mine_ec.EngineConfig.from_env()), flat(their_ec.EngineConfig.from_env())
    assert {k for k in fb if fa.get(k) != fb[k]} <= {"backends.attn", "backends.norm"}


def test_cosmos3_generation_media_output(ref):
    from phyai_b200.tools import cosmos3 as mine

    theirs = ref("phyai_utils_tools.models.cosmos3.processor_cosmos3")
    g = torch.Generator().manual_seed(0)
    video = torch.rand(1, 3, 5, 16, 24, generator=g) * 1.2 - 0.1           # a little outside [0, 1]: clamped
    sound = torch.randn(1, 2, 480, generator=g)
    a, b = mine.Cosmos3GenerationPostProcessor(fps=24), theirs.Cosmos3GenerationPostProcessor(fps=24)
    for out in (video, video[0], {"video": video, "sound": sound, "sample_rate": 48000}):
        x, y = a.postprocess(out), b.postprocess(out)
        assert torch.equal(x.frames, y.frames) and x.frames.dtype == torch.uint8 and torch.equal(x.video, y.video)
        assert (x.waveform is None) == (y.waveform is None) and (x.waveform is None or torch.equal(x.waveform, y.waveform))
        assert x.sample_rate == y.sample_rate and x["frames"] is x.frames
    for bad in (torch.rand(3, 16, 24), torch.rand(1, 4, 5, 16, 24)):
        with pytest.raises(ValueError):
            a.postprocess(bad)
        with pytest.raises(ValueError):
            b.postprocess(bad)


@pytest.mark.parametrize("variant", ["video", "action", "sound"])
def test_cosmos3_rotary_tables_for_text_video_action_and_sound_tokens(ref_single_rank, variant):
    """Positions of a whole request (text with padding, video grid rescaled by the frame rate, action tokens one frame
    later at their own rate, sound tokens at the sound rate) turned into cos / sin tables by both packages' transformers."""
    from phyai_b200 import parallel as P
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.models.cosmos3 import Cosmos3Transformer, tiny_cosmos3_config

    ref = ref_single_rank
    rm = ref("phyai.models.cosmos3.modeling_cosmos3")
    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    P.init((1,), ("tp",), device="cpu")
    try:
        cfg = tiny_cosmos3_config(action_gen=variant == "action", sound_gen=variant == "sound")
        mine = Cosmos3Transformer(cfg, params_dtype=torch.float32, device="cpu")
        theirs = rm.Cosmos3Transformer(_mirror_config(cfg, rm), params_dtype=torch.float32, device="cpu")
        mask = torch.tensor([[1, 1, 1, 1, 1, 0, 0], [1, 1, 1, 0, 0, 0, 0]])          # two prompts of different length, right-padded
        for fps, sfps in ((None, None), (24.0, 25.0), (10.0, 50.0)):
            kw = dict(action_len=5 if variant == "action" else 0, sound_len=7 if variant == "sound" else 0, sound_fps=sfps if variant == "sound" else None)
            und, gen = mine._rope_tables(mask, 3, 2, 3, fps, "cpu", **kw)
            (cu, su), (cg, sg) = theirs._compute_rope_freqs(mask, 3, 2, 3, fps, torch.device("cpu"), torch.float32, **kw)
            half = cfg.head_dim // 2
            for got, cos, sin, what in ((und, cu, su, "text"), (gen, cg, sg, "generated")):
                assert got.shape[:2] == cos.shape[:2], (variant, fps, what)
                assert torch.allclose(got[..., :half], cos[:, :, 0, :half], atol=1e-5), (variant, fps, what)
                assert torch.allclose(got[..., half:], sin[:, :, 0, :half], atol=1e-5), (variant, fps, what)
    finally:
        P.shutdown()


def test_cosmos3_adapters_around_the_decoder_stack(ref_single_rank, tmp_path):
    """The pieces of the Cosmos3 transformer that are plain tensor code in the reference too, run with the same weights:
    latent <-> token reshapes (grid sizes that need padding included), the timestep embedding, the per-domain action
    projections and the gate that keeps the timestep off clean frames."""
    from phyai_b200 import parallel as P
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.models.cosmos3 import Cosmos3Transformer, tiny_cosmos3_config
    from phyai_b200.models.cosmos3.transformer_cosmos3 import cosmos3_inverse_remap, cosmos3_weight_remap
    from phyai_b200.weights import load_pretrained, synthetic_state_dict, write_checkpoint

    ref = ref_single_rank
    rm = ref("phyai.models.cosmos3.modeling_cosmos3")
    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    P.init((1,), ("tp",), device="cpu")
    try:
        cfg = tiny_cosmos3_config(action_gen=True)
        mine = Cosmos3Transformer(cfg, params_dtype=torch.float32, device="cpu")
        theirs = rm.Cosmos3Transformer(_mirror_config(cfg, rm), params_dtype=torch.float32, device="cpu")
        g = torch.Generator().manual_seed(5)
        state = {cosmos3_inverse_remap(k): torch.randn(v.shape, generator=g) * 0.1 for k, v in synthetic_state_dict(mine, seed=1, std=0.05).items()}
        write_checkpoint(tmp_path, state, None)
        ref("phyai.weights.loader").load_pretrained(theirs, tmp_path, remap=rm.cosmos3_weight_remap, strict=True)
        load_pretrained(mine, tmp_path, remap=cosmos3_weight_remap, strict=True)

        c, p = cfg.latent_channel, cfg.latent_patch_size
        for t, h, w in ((2, 2 * p, 3 * p), (3, 2 * p + 1, 3 * p - 1), (1, 1, 1)):
            lat = torch.randn(2, c, t, h, w, generator=g)
            tok_m, tok_r = mine.patchify(lat, t, h, w), theirs.patchify(lat, t, h, w)
            assert torch.equal(tok_m, tok_r), (t, h, w)
            assert torch.equal(mine.unpatchify(tok_m, t, h, w), theirs.unpatchify(tok_r, t, h, w)), (t, h, w)
            assert torch.equal(mine.unpatchify(tok_m, t, h, w), lat), (t, h, w)
            assert mine._pad_to_patch_size(h, w) == theirs._pad_to_patch_size(h, w)

        ref("phyai.layers.linear").init(register_flashinfer=False, validate=False)      # its linears pick a kernel per call: the torch one
        ts = torch.tensor([0.0, 1.0, 37.5, 999.0])
        assert torch.allclose(mine.time_embedder(ts), theirs.time_embedder(ts), atol=1e-5, rtol=1e-5)

        dom = torch.tensor([0, cfg.num_embodiment_domains - 1, 1])
        act = torch.randn(3, 5, cfg.action_dim, generator=g)
        hid = torch.randn(3, 5, cfg.hidden_size, generator=g)
        assert torch.allclose(mine.action_proj_in(act, dom), theirs.action_proj_in(act, dom), atol=1e-6)
        assert torch.allclose(mine.action_proj_out(hid, dom), theirs.action_proj_out(hid, dom), atol=1e-6)
        assert torch.allclose(mine.action_proj_in(act[:, 0], dom), theirs.action_proj_in(act[:, 0], dom), atol=1e-6)

        emb = torch.randn(2, cfg.hidden_size, generator=g)
        frames = torch.tensor([[0.0, 1.0, 1.0], [1.0, 0.0, 1.0]])
        for mask in (None, frames):
            assert torch.equal(mine._gate_timestep(emb, mask, 4), theirs._gate_timestep(emb, mask, 4))
    finally:
        ref("phyai.layers.linear")._reset_for_test()
        P.shutdown()


def test_pi05_embeddings_and_heads(ref_single_rank, tmp_path):
    """The ends of the Pi0.5 network that are plain tensor code in the reference too, with the same weights: patch and
    position embedding of the cameras, scaled token embedding of the prompt, the flow-time embedding that conditions the
    action expert's norms, and the action projections in and out."""
    from phyai_b200 import parallel as P
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.models.pi05.configuration_pi05 import tiny_pi05_config
    from phyai_b200.models.pi05.modeling_pi05 import PI05Model
    from phyai_b200.weights import load_pretrained, synthetic_state_dict, write_checkpoint

    ref = ref_single_rank
    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    P.init((1,), ("tp",), device="cpu")
    try:
        cfg = tiny_pi05_config()
        mine = PI05Model(cfg)
        theirs = ref("phyai.models.pi05.modeling_pi05").PI05Model(_mirror_config(cfg, ref("phyai.models.pi05.configuration_pi05")),
                                                                  attn_backend="flashinfer", norm_backend="flashinfer", device="cpu")
        ref("phyai.engine")
        g = torch.Generator().manual_seed(9)
        state = {k: torch.randn(v.shape, generator=g) * 0.1 for k, v in synthetic_state_dict(mine, seed=1, std=0.05).items()}
        write_checkpoint(tmp_path, state, None)
        ref("phyai.weights.loader").load_pretrained(theirs, tmp_path, remap=ref("phyai.models.pi05.main_pi05")._compose_remap(None), strict=True)
        load_pretrained(mine, tmp_path, strict=True)
        ref("phyai.layers.linear").init(register_flashinfer=False, validate=False)

        v = cfg.vision
        pix = torch.rand(2, v.num_channels, v.image_size, v.image_size, generator=g) * 2 - 1
        assert torch.allclose(mine.vision.embed_patches(pix), theirs.vision.vision_tower.vision_model.embeddings(pix), atol=1e-5)

        ids = torch.randint(0, cfg.text.vocab_size, (2, 7), generator=g)
        assert torch.allclose(mine.paligemma_lm.embed_lang(ids), theirs.paligemma_lm.embed_lang(ids), atol=1e-6)

        t = torch.tensor([1.0, 0.9, 0.35, 0.0])
        assert torch.allclose(mine.heads.embed_time(t), theirs.heads.embed_time(t), atol=1e-5)

        noise = torch.randn(2, cfg.chunk_size, cfg.max_action_dim, generator=g)
        hid = torch.randn(2, cfg.chunk_size, cfg.expert.hidden_size, generator=g)
        assert torch.allclose(mine.heads.action_in_proj(noise)[0], theirs.heads.embed_action(noise), atol=1e-5)
        assert torch.allclose(mine.heads.action_out_proj(hid)[0], theirs.heads.project_action(hid), atol=1e-5)
    finally:
        ref("phyai.layers.linear")._reset_for_test()
        P.shutdown()


def test_pi0_state_and_action_time_heads(ref_single_rank, tmp_path):
    """Pi0 feeds the robot state as one token and mixes the flow time into every action token through a small network
    (no time-conditioned norms): both, and the projection back to actions, with the same weights in both packages."""
    from phyai_b200 import parallel as P
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.models.pi0.configuration_pi0 import tiny_pi0_config
    from phyai_b200.models.pi0.modeling_pi0 import PI0Model
    from phyai_b200.weights import load_pretrained, synthetic_state_dict, write_checkpoint

    ref = ref_single_rank
    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    P.init((1,), ("tp",), device="cpu")
    try:
        cfg = tiny_pi0_config()
        mine = PI0Model(cfg)
        theirs = ref("phyai.models.pi0.modeling_pi0").PI0Model(_mirror_config(cfg, ref("phyai.models.pi0.configuration_pi0")),
                                                               attn_backend="flashinfer", norm_backend="flashinfer", device="cpu")
        ref("phyai.engine")
        g = torch.Generator().manual_seed(11)
        state = {k: torch.randn(v.shape, generator=g) * 0.1 for k, v in synthetic_state_dict(mine, seed=1, std=0.05).items()}
        write_checkpoint(tmp_path, state, None)
        ref("phyai.weights.loader").load_pretrained(theirs, tmp_path, remap=ref("phyai.models.pi0.main_pi0")._compose_remap(None), strict=True)
        load_pretrained(mine, tmp_path, strict=True)
        ref("phyai.layers.linear").init(register_flashinfer=False, validate=False)

        robot = torch.randn(1, cfg.max_state_dim, generator=g)
        assert torch.allclose(mine.heads.state_proj(robot)[0], theirs.heads.embed_state(robot), atol=1e-5)
        x_t = torch.randn(cfg.chunk_size, cfg.max_action_dim, generator=g)
        for t in (1.0, 0.6, 0.1):
            got = mine.heads.embed_action_time(x_t, torch.tensor([t]))
            want = theirs.heads.embed_action_time(x_t[None], torch.tensor([t]))[0]
            assert torch.allclose(got, want, atol=1e-5), t
        hid = torch.randn(cfg.chunk_size, cfg.expert.hidden_size, generator=g)
        assert torch.allclose(mine.heads.action_out_proj(hid)[0], theirs.heads.project_action(hid[None])[0], atol=1e-5)
        ids = torch.randint(0, cfg.text.vocab_size, (1, 6), generator=g)
        assert torch.allclose(mine.paligemma_lm.embed_lang(ids), theirs.paligemma_lm.embed_lang(ids), atol=1e-6)
    finally:
        ref("phyai.layers.linear")._reset_for_test()
        P.shutdown()


class _StubDenoiser:
    """Stands in for the network inside both packages' Cosmos3 schedulers: a closed-form "velocity" of everything the
    loop hands it (latents, timestep, prompt, masks, domain), so the loops can be compared without a GPU."""

    use_cuda_graph = False

    def __init__(self):
        self.calls = []

    def setup(self):
        pass

    def reset(self, held=None):
        self.calls.append("reset")

    def prepare(self, branch, **kw):
        pass

    def forward(self, branch, video, t, *, text_ids, text_mask, video_shape, fps, noisy_frame_mask=None, action_latents=None,
                action_domain_id=None, action_noisy_mask=None, sound_latents=None, sound_fps=None):
        self.calls.append(branch)
        s = 1.0 if branch == "cond" else 0.55
        bias = 1e-3 * float(t.float().reshape(-1)[0]) + 1e-2 * float((text_ids * text_mask).float().mean()) / 100.0 + 1e-3 * fps / 24.0
        v = torch.tanh(video.float() * s) * 0.7 + bias
        if noisy_frame_mask is not None:
            v = v * (0.5 + 0.5 * noisy_frame_mask.float())[:, None, :, None, None]
        if action_latents is not None:
            a = torch.sin(action_latents.float() * s) + bias + 0.01 * action_domain_id.float()[:, None, None]
            a = a * (0.25 + 0.75 * action_noisy_mask.float())[..., None] + 0.05 * v.mean()
            return v.to(video.dtype), a.to(action_latents.dtype)
        if sound_latents is not None:
            return v.to(video.dtype), (torch.cos(sound_latents.float()) * s + bias * sound_fps / 25.0).to(sound_latents.dtype)
        return v.to(video.dtype)


def _tiny_prompts(g, B=1):
    ids = torch.randint(1, 90, (B, 6), generator=g)
    mask = torch.tensor([[1, 1, 1, 1, 0, 0]] * B)
    nids = torch.randint(1, 90, (B, 6), generator=g)
    nmask = torch.tensor([[1, 1, 1, 0, 0, 0]] * B)
    return dict(text_ids=ids, text_mask=mask, neg_text_ids=nids, neg_text_mask=nmask)


@pytest.mark.parametrize("case", ["t2v", "t2v_noguide", "i2v", "sound", "given_noise"])
def test_cosmos3_generation_loop_around_a_stub_network(ref_single_rank, case):
    """The whole denoise loop of the generation scheduler (seeded noise, guidance mix, one solver per stream, clean frames
    written back after every step, sound layout on return) run in both packages around the same stand-in network."""
    from phyai_b200 import parallel as P
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.models.cosmos3 import Cosmos3Transformer, tiny_cosmos3_config
    from phyai_b200.models.cosmos3.scheduler_cosmos3 import Cosmos3T2VRequest, Cosmos3T2VScheduler

    ref = ref_single_rank
    rm, rs = ref("phyai.models.cosmos3.modeling_cosmos3"), ref("phyai.models.cosmos3.scheduler_ws1_cosmos3")
    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    P.init((1,), ("tp",), device="cpu")
    try:
        cfg = tiny_cosmos3_config(sound_gen=case == "sound")
        mine = Cosmos3T2VScheduler(Cosmos3Transformer(cfg, params_dtype=torch.float32, device="cpu"), device="cpu", flow_shift=3.0, use_karras_sigmas=False)
        theirs = rs.Cosmos3T2VScheduler(rm.Cosmos3Transformer(_mirror_config(cfg, rm), params_dtype=torch.float32, device="cpu"), device="cpu",
                                        flow_shift=3.0, use_karras_sigmas=False)
        mine.setup()
        mine.runner, theirs.runner = _StubDenoiser(), _StubDenoiser()
        theirs.setup()
        g = torch.Generator().manual_seed(3)
        t, h, w = 3, 4, 6
        kw = dict(_tiny_prompts(g), video_shape=(t, h, w), fps=16.0, num_inference_steps=6, guidance_scale=1.0 if case == "t2v_noguide" else 4.5, seed=7)
        if case == "i2v":
            kw.update(cond_latents=torch.randn(1, cfg.latent_channel, t, h, w, generator=g), cond_frame_indexes=(0, 2))
        if case == "sound":
            kw.update(sound_frames=9, sound_dim=cfg.sound_dim, sound_latent_fps=25.0)
        if case == "given_noise":
            kw.update(noise=torch.randn(1, cfg.latent_channel, t, h, w, generator=g))
        got, want = mine.step(Cosmos3T2VRequest(**kw)), theirs.step(rs.Cosmos3T2VRequest(**kw))
        assert mine.runner.calls == theirs.runner.calls and len(mine.runner.calls) == 1 + 6 * (1 if case == "t2v_noguide" else 2)
        if case == "sound":
            assert got["sound"].shape == want["sound"].shape == (1, cfg.sound_dim, 9)
            assert torch.allclose(got["sound"], want["sound"], atol=2e-5)
            got, want = got["video"], want["video"]
        assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
        if case == "i2v":
            assert torch.equal(got[:, :, [0, 2]], kw["cond_latents"][:, :, [0, 2]])
    finally:
        P.shutdown()


@pytest.mark.parametrize("mode,guide,batch,frames", [("policy", 1.0, 1, None), ("policy", 3.0, 2, None), ("forward_dynamics", 1.0, 1, None),
                                                     ("inverse_dynamics", 2.0, 1, None), ("policy", 1.0, 1, (0, 1))])
def test_cosmos3_policy_loop_around_a_stub_network(ref_single_rank, mode, guide, batch, frames):
    """The joint video + action loop in its three modes: which frames and which stream stay clean, the zeroed tail beyond
    the robot's action width, per-sample noise in a batch, guidance on both streams, in both packages around one stub."""
    from phyai_b200 import parallel as P
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.models.cosmos3 import Cosmos3Transformer, tiny_cosmos3_config
    from phyai_b200.models.cosmos3.scheduler_cosmos3 import Cosmos3ActionRequest, Cosmos3PolicyScheduler

    ref = ref_single_rank
    rm, rs = ref("phyai.models.cosmos3.modeling_cosmos3"), ref("phyai.models.cosmos3.scheduler_ws1_cosmos3_policy")
    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    P.init((1,), ("tp",), device="cpu")
    try:
        cfg = tiny_cosmos3_config(action_gen=True)
        mine = Cosmos3PolicyScheduler(Cosmos3Transformer(cfg, params_dtype=torch.float32, device="cpu"), device="cpu", flow_shift=2.0, use_karras_sigmas=True)
        theirs = rs.Cosmos3PolicyScheduler(rm.Cosmos3Transformer(_mirror_config(cfg, rm), params_dtype=torch.float32, device="cpu"), device="cpu",
                                           flow_shift=2.0, use_karras_sigmas=True, use_cuda_graph=False)
        mine.setup()
        mine.runner, theirs.runner = _StubDenoiser(), _StubDenoiser()
        theirs.setup()
        g = torch.Generator().manual_seed(4)
        t, h, w, chunk, raw = 3, 4, 4, 5, 7
        kw = dict(_tiny_prompts(g, batch), video_shape=(t, h, w), mode=mode, domain_id=2, action_chunk=chunk, raw_action_dim=raw, action_dim=cfg.action_dim,
                  cond_video_latents=torch.randn(batch, cfg.latent_channel, t, h, w, generator=g), cond_action=torch.randn(batch, chunk, cfg.action_dim, generator=g),
                  cond_frame_indexes=frames, fps=10.0, num_inference_steps=5, guidance_scale=guide, seed=11)
        got, want = mine.step(Cosmos3ActionRequest(**kw)), theirs.step(rs.Cosmos3ActionRequest(**kw))
        assert mine.runner.calls == theirs.runner.calls
        assert got["action"].shape == want["action"].shape == (batch, chunk, raw)
        assert torch.allclose(got["action"], want["action"], atol=2e-5), float((got["action"] - want["action"]).abs().max())
        assert torch.allclose(got["video"], want["video"], atol=2e-5), float((got["video"] - want["video"]).abs().max())
        if mode == "forward_dynamics":
            assert torch.equal(got["action"], kw["cond_action"][:, :, :raw])
        if mode == "inverse_dynamics":
            assert torch.equal(got["video"], kw["cond_video_latents"])
        if batch > 1 and mode == "policy":
            assert not torch.equal(got["action"][0], got["action"][1])
    finally:
        P.shutdown()


def test_tensor_dump_files_have_the_same_keys_and_values(ref, tmp_path):
    """One module tree (a module that returns a ``(tensor, None)`` pair, one called twice, one returning no tensor)
    hooked by both packages' dumpers through the reference's call: the pass files hold the same names and tensors, so a
    dump taken with one package can be compared key by key with a dump of the other."""
    from collections import OrderedDict

    from phyai_b200.runtime import tensor_dump as mine_mod

    ref_mod = ref("phyai.runtime.tensor_dump")

    class Pair(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.eye(4) * 2)

        def forward(self, x):
            return x @ self.w, None

    class Silent(torch.nn.Module):
        def forward(self, x):
            return "nothing to keep"

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.body = torch.nn.Sequential(OrderedDict(lin=torch.nn.Linear(4, 4), act=torch.nn.Tanh()))
            self.pair, self.silent = Pair(), Silent()

        def forward(self, x):
            y = self.body(x)
            y = self.body.act(y)
            self.silent(y)
            return self.pair(y)[0]

    torch.manual_seed(0)
    net, x = Net(), torch.randn(3, 4)
    results = {}
    for tag, mod in (("mine", mine_mod), ("theirs", ref_mod)):
        for flt in (None, [r"body\.", r"^net\.pair$"], lambda name, module: isinstance(module, torch.nn.Tanh)):
            d = mod.register_tensor_dumper({"net": net}, dump_dir=tmp_path / tag / str(len(results)), filter=flt, rank=3, world_size=4)
            net(x)
            first = d.flush_pass()
            net(x * 2)
            second = d.flush_pass()
            assert d.flush_pass() is None
            d.detach()
            assert first.parent == d.process_dir and first.parent.name.startswith("rank3_pid") and second.name == "pass00001.pt"
            results.setdefault(tag, []).append((mod.load_pass(first), mod.load_pass(second)))
    for (m1, m2), (t1, t2) in zip(results["mine"], results["theirs"]):
        for a, b in ((m1, t1), (m2, t2)):
            assert list(a) == list(b)
            assert all(torch.equal(a[k], b[k]) for k in a)
    everything = results["mine"][0][0]
    assert list(everything) == ["net.body.lin", "net.body.act", "net.body.act::call1", "net.pair"] and isinstance(everything["net.pair"], torch.Tensor)
    assert list(results["mine"][2][0]) == ["net.body.act", "net.body.act::call1"]
    with pytest.raises(TypeError):
        mine_mod.TensorDumper({"net": net}, dump_dir=tmp_path / "bad", filter="net")
    with pytest.raises(ValueError):
        mine_mod.TensorDumper({}, dump_dir=tmp_path / "bad")
