"""Cosmos3 prompt / bucket helpers and policy-mode steps one by one (the end-to-end processor is covered in test_tools.py)."""

import json

import numpy as np
import pytest
import torch

from phyai_b200.tools import cosmos3 as c3
from phyai_b200.tools.processing import IMAGES, PIXEL_VALUES


def test_resolution_tables_are_consistent():
    for tier, buckets in c3.VIDEO_RES_SIZE_INFO.items():
        assert set(buckets) == {"1,1", "4,3", "3,4", "16,9", "9,16"}
        for ar, (w, h) in buckets.items():
            assert w % 8 == 0 and h % 8 == 0, (tier, ar)                            # whole latent pixels (the VAE shrinks by 8)
            aw, ah = (int(x) for x in ar.split(","))
            assert abs((w / h) / (aw / ah) - 1) < 0.09, (tier, ar)                   # the bucket has about the aspect it is named for
            assert c3.aspect_ratio_str(w, h) == ar
            tw, th = buckets[f"{ah},{aw}"]
            assert (tw, th) == (h, w)                                                # portrait is landscape transposed
    assert set(c3.EMBODIMENT_TO_RAW_ACTION_DIM) <= set(c3.EMBODIMENT_TO_DOMAIN_ID)


@pytest.mark.parametrize("h,w,tier,want", [(720, 1280, "480", (832, 480)), (1280, 720, "480", (480, 832)), (500, 500, "256", (256, 256)),
                                            (600, 800, 704, (1088, 832)), (1080, 1920, "1080", (1920, 1080)), (100, 100, "gt_2048", (5464, 5464))])
def test_closest_bucket_by_aspect(h, w, tier, want):
    assert c3.find_closest_target_size(h, w, tier) == want                          # (width, height)


def test_tier_of_a_frame_and_target_of_an_observation():
    assert [c3.get_vision_data_resolution(s) for s in ((256, 400), (480, 640), (640, 1000), (720, 1280), (960, 960))] == ["256", "480", "480", "720", "720"]
    assert c3.get_vision_data_resolution((768, 1360)) == "768" and c3.get_vision_data_resolution((880, 1184)) == "768"   # exact 768-tier shapes
    with pytest.raises(ValueError, match="no resolution tier"):
        c3.get_vision_data_resolution((1080, 1920))
    assert c3.resolve_target_size(720, 1280, 480) == (480, 832)                     # (height, width): 16:9 at 480 rows
    assert c3.resolve_target_size(480, 640, 224) == (256, 320)                      # 4:3 at 224 rows: the 256 tier
    assert c3.resolve_target_size(1000, 500, 480) == (320, 192)                     # portrait: 240 columns at 480 rows is the 256 tier


def test_bucket_and_aspect_errors():
    with pytest.raises(ValueError, match="unknown resolution tier"):
        c3.find_closest_target_size(10, 10, "999")
    assert set(c3.VIDEO_RES_SIZE_INFO) == {"256", "480", "704", "720", "768", "1080", "1280", "2048", "gt_2048"}
    with pytest.raises(ValueError, match="non-zero"):
        c3.aspect_ratio_str(0, 0)
    assert c3.aspect_ratio_str(1920, 1200) == "8,5"                                 # not a bucket: the reduced fraction
    with pytest.raises(ValueError, match="non-negative"):
        c3.resolve_domain_id(-1)
    assert c3.resolve_domain_id("  Droid_LeRobot ") == 8 and c3.resolve_raw_action_dim("AgiBotWorld") == 29
    with pytest.raises(ValueError, match="no action width on record"):
        c3.resolve_raw_action_dim("libero")


def test_action_caption_fields_and_punctuation():
    a = json.loads(c3.cosmos3_action_json_caption("Pick the cup!", view_point="wrist_view", num_frames=125, fps=10, height=480, width=832))
    assert "wrist-mounted camera" in a["cinematography"]["framing"] and a["actions"][0] == {"time": "0:00-0:12", "description": "Pick the cup!"}
    assert a["duration"] == "12s" and a["fps"] == 10.0 and a["resolution"] == {"H": 480, "W": 832}
    b = json.loads(c3.cosmos3_action_json_caption("walk", view_point="unknown_view", num_frames=700, fps=10, height=100, width=150))
    assert "cinematography" not in b and b["actions"][0] == {"time": "0:00-1:10", "description": "walk."} and b["aspect_ratio"] == "3,2"
    assert list(b) == ["actions", "duration", "fps", "resolution", "aspect_ratio"]   # key order is part of the prompt


def test_generation_caption_text_and_json_forms():
    still = c3.cosmos3_generation_caption("A cat.", fps=24, num_frames=1, height=480, width=832)
    assert still == "A cat. This video is of 480x832 resolution."                   # a still gets no duration sentence
    clip = json.loads(c3.cosmos3_generation_caption('{"scene": "lab", "duration": "9s"}', fps=16, num_frames=81, height=704, width=1280))
    assert clip == {"scene": "lab", "duration": "5s", "fps": 16.0, "resolution": {"H": 704, "W": 1280}}
    one = json.loads(c3.cosmos3_generation_caption('{"scene": "lab", "duration": "9s", "fps": 3}', fps=16, num_frames=1, height=8, width=8))
    assert "duration" not in one and "fps" not in one
    assert c3.cosmos3_generation_caption("[1, 2]", fps=10, num_frames=1, height=8, width=8).startswith("[1, 2].")   # JSON, but not an object
    neg = json.loads(c3.cosmos3_default_negative_prompt())
    assert "artifacts" in neg and isinstance(neg["artifacts"], list)


def test_image_step_targets_inputs_and_margins():
    snap = c3.Cosmos3ImagePreprocessStep(height=1, width=1, mode="policy", image_size=256)
    arr = (np.random.rand(90, 160, 3) * 255).astype("uint8")
    t = snap({IMAGES: arr})
    assert t[PIXEL_VALUES].shape == (1, 3, 1, 192, 320) and t[c3.VIDEO_SHAPE] == (1, 192, 320)                 # the 16:9 bucket of the 256 tier
    assert (t[c3.META_HEIGHT], t[c3.META_WIDTH]) == (256, 455)                                                 # the frame scaled to 256 rows
    assert torch.equal(t[PIXEL_VALUES][0, :, 0, :90, :160], torch.from_numpy(arr).permute(2, 0, 1).float() / 127.5 - 1.0)   # never enlarged
    fixed = c3.Cosmos3ImagePreprocessStep(height=32, width=48, mode="inverse_dynamics")
    frames = [torch.rand(3, 64, 96), np.random.rand(64, 96, 3).astype("float32") * 2 - 1, (np.random.rand(3, 64, 96) * 255).astype("uint8")]
    t2 = fixed({IMAGES: frames})
    assert t2[PIXEL_VALUES].shape == (1, 3, 3, 32, 48) and t2[c3.VIDEO_SHAPE] == (3, 32, 48) and (t2[c3.META_HEIGHT], t2[c3.META_WIDTH]) == (32, 48)
    assert float(t2[PIXEL_VALUES].abs().max()) <= 1.0
    assert fixed.get_config() == {"height": 32, "width": 48, "mode": "inverse_dynamics", "image_size": None}
    with pytest.raises(ValueError, match="needs 'images'"):
        fixed({})
    # margins: reflected while they are narrower than the picture, the edge repeated otherwise
    ramp = np.tile(np.arange(8, dtype=np.uint8)[None, :, None] * 30, (4, 1, 3))
    out = c3.resize_and_pad_action_image(ramp, 4, 12)
    assert out.shape == (4, 12, 3) and out[0, :, 0].tolist() == [0, 30, 60, 90, 120, 150, 180, 210, 180, 150, 120, 90]
    out = c3.resize_and_pad_action_image(ramp, 4, 20)
    assert out[0, 8:, 0].tolist() == [210] * 12
    with pytest.raises(TypeError, match="an image is"):
        c3.resize_and_pad_action_image([1, 2, 3], 4, 4)


def test_action_pad_step_modes():
    pad = c3.Cosmos3ActionPadStep(action_chunk_size=4, raw_action_dim=3, action_dim=8, mode="forward_dynamics")
    t = pad({c3.COND_ACTION: np.arange(6, dtype="float32").reshape(2, 3)})
    a = t[c3.COND_ACTION]
    assert a.shape == (1, 4, 8) and a[0, :, :3].tolist() == [[0, 1, 2], [3, 4, 5], [3, 4, 5], [3, 4, 5]] and a[0, :, 3:].abs().sum() == 0
    long = pad({c3.COND_ACTION: torch.ones(1, 9, 3)})[c3.COND_ACTION]
    assert long.shape == (1, 4, 8)                                                  # cut to the chunk
    assert (t[c3.ACTION_CHUNK], t[c3.RAW_ACTION_DIM], t[c3.MODE]) == (4, 3, "forward_dynamics")
    assert pad({c3.COND_ACTION: torch.ones(2, 3), c3.MODE: "given"})[c3.MODE] == "given"        # a mode set upstream is kept
    with pytest.raises(ValueError, match="needs 'cond_action'"):
        pad({})
    pol = c3.Cosmos3ActionPadStep(action_chunk_size=4, raw_action_dim=3, mode="policy")({c3.COND_ACTION: torch.ones(2, 3)})
    assert pol[c3.COND_ACTION] is None and pol[c3.MODE] == "policy"                 # a policy request carries no conditioning action


def test_domain_step():
    assert c3.Cosmos3DomainResolveStep()({c3.DOMAIN_ID: "fractal"})[c3.DOMAIN_ID] == 20
    assert c3.Cosmos3DomainResolveStep()({c3.DOMAIN_ID: 11})[c3.DOMAIN_ID] == 11
    with pytest.raises(ValueError, match="needs 'domain_id'"):
        c3.Cosmos3DomainResolveStep()({})
