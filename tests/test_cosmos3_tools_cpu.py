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


@pytest.mark.parametrize("h,w,tier,want", [(720, 1280, "480", (480, 832)), (1280, 720, "480", (832, 480)), (500, 500, "256", (256, 256)),
                                            (600, 800, 704, (832, 1088)), (1080, 1920, "1080", (1080, 1920))])
def test_closest_bucket_by_aspect(h, w, tier, want):
    assert c3.find_closest_target_size(h, w, tier) == want


def test_bucket_and_aspect_errors():
    with pytest.raises(ValueError, match="unknown resolution tier"):
        c3.find_closest_target_size(10, 10, "999")
    with pytest.raises(ValueError, match="non-zero"):
        c3.aspect_ratio_str(0, 0)
    assert c3.aspect_ratio_str(1920, 1200) == "8,5"                                 # not a bucket: the reduced fraction
    with pytest.raises(ValueError, match="non-negative"):
        c3.resolve_domain_id(-1)
    assert c3.resolve_domain_id("  Droid_LeRobot ") == 8 and c3.resolve_raw_action_dim("AgiBotWorld") == 29
    with pytest.raises(ValueError, match="no action width on record"):
        c3.resolve_raw_action_dim("libero")


def test_action_caption_fields_and_punctuation():
    a = json.loads(c3.cosmos3_action_json_caption("Pick the cup!", view_point="wrist", num_frames=125, fps=10, height=480, width=832))
    assert a["cinematography"]["framing"].startswith("close-up") and a["actions"][0] == {"time": "0:00-0:12", "description": "Pick the cup!"}
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


def test_image_step_accepts_arrays_tensors_and_lists():
    step = c3.Cosmos3ImagePreprocessStep(resolution="256", action_chunk_size=16)
    arr = (np.random.rand(90, 160, 3) * 255).astype("uint8")
    t = step({IMAGES: arr})
    assert t[PIXEL_VALUES].shape == (1, 3, 1, 192, 320) and -1.0 <= float(t[PIXEL_VALUES].min()) and float(t[PIXEL_VALUES].max()) <= 1.0
    assert t[c3.VIDEO_SHAPE] == (5, 12, 20) and (t[c3.META_HEIGHT], t[c3.META_WIDTH]) == (180, 320)
    chw = torch.rand(3, 64, 64)
    t2 = step({IMAGES: [chw]})
    assert t2[PIXEL_VALUES].shape == (1, 3, 1, 256, 256) and t2[c3.VIDEO_SHAPE] == (5, 16, 16)
    assert step.get_config() == {"resolution": "256", "temporal": 4, "spatial": 16, "action_chunk_size": 16}


def test_action_pad_step_modes():
    pad = c3.Cosmos3ActionPadStep(action_chunk_size=4, raw_action_dim=3, action_dim=8, mode="forward_dynamics")
    t = pad({c3.COND_ACTION: np.arange(6, dtype="float32").reshape(2, 3)})
    a = t[c3.COND_ACTION]
    assert a.shape == (1, 4, 8) and a[0, :, :3].tolist() == [[0, 1, 2], [3, 4, 5], [3, 4, 5], [3, 4, 5]] and a[0, :, 3:].abs().sum() == 0
    long = pad({c3.COND_ACTION: torch.ones(1, 9, 3)})[c3.COND_ACTION]
    assert long.shape == (1, 4, 8)                                                  # cut to the chunk
    assert (t[c3.ACTION_CHUNK], t[c3.RAW_ACTION_DIM], t[c3.MODE]) == (4, 3, "forward_dynamics")
    with pytest.raises(ValueError, match="needs 'cond_action'"):
        pad({})
    pol = c3.Cosmos3ActionPadStep(action_chunk_size=4, raw_action_dim=3, mode="policy")({c3.COND_ACTION: torch.ones(2, 3)})
    assert pol[c3.COND_ACTION] is None and pol[c3.MODE] == "policy"                 # a policy request carries no conditioning action


def test_domain_step():
    assert c3.Cosmos3DomainResolveStep()({c3.DOMAIN_ID: "fractal"})[c3.DOMAIN_ID] == 20
    assert c3.Cosmos3DomainResolveStep()({c3.DOMAIN_ID: 11})[c3.DOMAIN_ID] == 11
    with pytest.raises(ValueError, match="needs 'domain_id'"):
        c3.Cosmos3DomainResolveStep()({})
