import json
from dataclasses import dataclass, field

import pytest

from phyai_b200.models.configuration import PretrainedConfig
from phyai_b200.models.pi05.configuration_pi05 import PI05Config, SiglipVisionConfig, tiny_pi05_config


@dataclass(frozen=True)
class Inner(PretrainedConfig):
    width: int = 4
    shape: tuple[int, ...] = (1, 2)


@dataclass(frozen=True)
class Outer(PretrainedConfig):
    nested_sources = {"depth": "arch.depth"}
    inner: Inner = field(default_factory=Inner)
    depth: int = 1
    name: str = "x"


def test_from_dict_drops_unknown_and_recurses():
    o = Outer.from_dict({"inner": {"width": 8, "shape": [3, 4], "junk": 1}, "arch": {"depth": 7}, "zzz": 0})
    assert o.inner.width == 8 and o.inner.shape == (3, 4) and o.depth == 7 and o.name == "x"


def test_mapping_access_and_roundtrip(tmp_path):
    o = Outer(depth=3)
    assert o["depth"] == 3 and "inner" in o and o.get("nope", 5) == 5
    with pytest.raises(KeyError):
        o["nope"]
    p = tmp_path / "config.json"
    o.to_json(p)
    assert Outer.from_json(p) == o
    assert json.loads(p.read_text())["inner"]["shape"] == [1, 2]


def test_pi05_config_validation():
    c = PI05Config()
    assert c.vision.num_patches == 256 and c.vision.head_dim == 72 and c.num_layers == 18
    with pytest.raises(ValueError):
        SiglipVisionConfig(image_size=225)
    with pytest.raises(ValueError):
        PI05Config(vision=SiglipVisionConfig(projection_dim=1024))
    t = tiny_pi05_config()
    assert PI05Config.from_dict(t.to_dict()) == t
