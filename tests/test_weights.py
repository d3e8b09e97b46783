import json

import pytest
import torch
import torch.nn as nn
from safetensors.torch import save_file

from phyai_b200.parallel.mesh import Mesh
from phyai_b200.weights import load_pretrained, shards, synthetic_state_dict, write_checkpoint


def fake_mesh(tp=4, rank=2):
    return Mesh((tp,), ("tp",), rank=rank, build_groups=False)


def P(*shape):
    return nn.Parameter(torch.zeros(*shape), requires_grad=False)


def test_sharded_dim0_tp4_rank2():
    p, full = P(2, 3), torch.arange(24.).reshape(8, 3)
    shards.sharded(0, "tp", fake_mesh())(p, full, None)
    assert torch.equal(p.data, full[4:6])


def test_sharded_dim1_and_replicate():
    p, full = P(3, 4), torch.arange(24.).reshape(3, 8)
    shards.sharded(1, "tp", fake_mesh(2, 1))(p, full, None)
    assert torch.equal(p.data, full[:, 4:])
    p2, kv = P(4, 2), torch.arange(16.).reshape(8, 2)
    shards.sharded(0, "tp", fake_mesh(4, 3), replicate=2)(p2, kv, None)   # ranks 2,3 share part 1
    assert torch.equal(p2.data, kv[4:])


def test_fused_qkv_layout_with_kv_replication():
    # 4 q heads, 1 kv head, head_dim 2, tp=2: each rank holds 2 q heads + the replicated kv head
    m = fake_mesh(2, 1)
    table = {"q": (0, 4), "k": (4, 2), "v": (6, 2)}
    ld = shards.fused(0, table, "tp", m, replicate={"q": 1, "k": 2, "v": 2})
    p = P(8, 3)
    q, k, v = torch.arange(24.).reshape(8, 3), torch.full((2, 3), 100.), torch.full((2, 3), 200.)
    ld(p, q, "q"); ld(p, k, "k"); ld(p, v, "v")
    assert torch.equal(p.data[:4], q[4:]) and torch.equal(p.data[4:6], k) and torch.equal(p.data[6:], v)
    with pytest.raises(KeyError):
        ld(p, q, "z")


def test_fused_interleave_gate_up():
    ld = shards.fused(0, {0: (0, 3), 1: (3, 3)}, None, None, interleave=True)
    p = P(6, 2)
    g, u = torch.ones(3, 2), torch.full((3, 2), 2.)
    ld(p, g, 0); ld(p, u, 1)
    assert torch.equal(p.data[0::2], g) and torch.equal(p.data[1::2], u)


def test_vocab_padding_zeros_trailing_rank():
    p = P(4, 2); p.data.fill_(9)
    shards.vocab(8, "tp", fake_mesh(2, 1))(p, torch.ones(6, 2), None)
    assert torch.equal(p.data[:2], torch.ones(2, 2)) and p.data[2:].abs().sum() == 0


def test_weight_norm_fold():
    ld = shards.weight_norm_fold(0)
    p = P(3, 4)
    v, g = torch.randn(3, 4), torch.rand(3, 1) + 0.5
    ld(p, g, "g"); ld(p, v, "v")
    assert torch.allclose(p.data, g * v / v.norm(dim=1, keepdim=True), atol=1e-6)


class Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(4, 3)
        self.b = P(2)
        self.b.hf_keys = {"renamed.b": None}
        self.c = P(2)
        self.c.hf_keys = {"opt.c": None}
        self.c.optional = True
        self.hooked = False

    def post_load(self):
        self.hooked = True


def _ckpt(tmp_path, extra=None, index=False):
    t = {"a.weight": torch.randn(3, 4), "a.bias": torch.randn(3), "renamed.b": torch.ones(2)}
    t.update(extra or {})
    if index:
        keys = list(t)
        save_file({k: t[k] for k in keys[:2]}, str(tmp_path / "model-00001-of-00002.safetensors"))
        save_file({k: t[k] for k in keys[2:]}, str(tmp_path / "model-00002-of-00002.safetensors"))
        wm = {k: ("model-00001-of-00002.safetensors" if i < 2 else "model-00002-of-00002.safetensors") for i, k in enumerate(keys)}
        (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    else:
        save_file(t, str(tmp_path / "model.safetensors"))
    return t


@pytest.mark.parametrize("index", [False, True])
def test_load_strict_ok_and_report(tmp_path, index):
    t = _ckpt(tmp_path, index=index)
    m = Toy()
    r = load_pretrained(m, tmp_path)
    assert torch.equal(m.a.weight.data, t["a.weight"]) and torch.equal(m.b.data, torch.ones(2))
    assert r.optional_missing == ["opt.c"] and not r.missing and not r.unexpected and m.hooked


def test_load_strict_fails_on_unexpected_and_missing(tmp_path):
    _ckpt(tmp_path, extra={"zzz": torch.zeros(1)})
    with pytest.raises(RuntimeError):
        load_pretrained(Toy(), tmp_path)
    r = load_pretrained(Toy(), tmp_path, strict=False)
    assert r.unexpected == ["zzz"]
    r = load_pretrained(Toy(), tmp_path, remap=lambda k: None if k == "zzz" else k)
    assert r.dropped == ["zzz"]
    r = load_pretrained(Toy(), tmp_path, remap={"zzz": None})
    assert r.dropped == ["zzz"]


def test_double_claim_is_an_error(tmp_path):
    _ckpt(tmp_path)
    m = Toy()
    m.c.hf_keys = {"renamed.b": None}
    with pytest.raises(ValueError):
        load_pretrained(m, tmp_path)


def test_synthetic_checkpoint_roundtrip(tmp_path):
    from phyai_b200.models.pi05.configuration_pi05 import tiny_pi05_config
    from phyai_b200.models.pi05.modeling_pi05 import PI05Model

    cfg = tiny_pi05_config()
    m = PI05Model(cfg)
    state = synthetic_state_dict(m, seed=1)
    assert any(k.endswith("q_proj.weight") for k in state) and any(k.endswith("gate_proj.weight") for k in state)
    write_checkpoint(tmp_path, state, cfg.to_dict(), shards=3)
    m2 = PI05Model(cfg)
    r = load_pretrained(m2, tmp_path)
    assert r.ok and len(r.loaded) == len(state)
    l0 = m2.paligemma_lm.layers[0]
    pre = "paligemma_with_expert.paligemma.model.language_model.layers.0"
    assert torch.equal(l0.mlp.gate_up.weight.data[0::2], state[f"{pre}.mlp.gate_proj.weight"])
    assert torch.equal(l0.attn.qkv.weight.data[-32:], state[f"{pre}.self_attn.v_proj.weight"])


# ---- the loader's public contract, as the reference states it (phyai/tests/weights/test_loader.py)
def _two_param_model():
    m = nn.Module()
    m.a = nn.Parameter(torch.zeros(2, 3), requires_grad=False)
    m.a.hf_keys = {"model.layers.0.a.weight": None}
    m.b = nn.Parameter(torch.zeros(4), requires_grad=False)      # no hf_keys: never "missing"
    return m


def test_dict_remap_is_an_ordered_substring_rewrite(tmp_path):
    from safetensors.torch import save_file

    from phyai_b200.weights.loader import load_pretrained

    f = tmp_path / "model.safetensors"
    save_file({"transformer.h.0.a.weight": torch.ones(2, 3), "transformer.drop.me": torch.zeros(1)}, str(f))
    m = _two_param_model()
    rep = load_pretrained(m, tmp_path, remap={"transformer.": "model.", ".h.": ".layers.", "drop.me": None})
    assert rep.ok and rep.loaded == ["model.layers.0.a.weight"] and rep.dropped == ["transformer.drop.me"]
    assert torch.equal(m.a, torch.ones(2, 3)) and "b" in rep.optional_missing


def test_source_may_be_one_file_or_a_list_of_files(tmp_path):
    from safetensors.torch import save_file

    from phyai_b200.weights.loader import load_pretrained

    f1, f2 = tmp_path / "part1.safetensors", tmp_path / "part2.safetensors"
    save_file({"model.layers.0.a.weight": torch.full((2, 3), 2.0)}, str(f1))
    save_file({"b": torch.full((4,), 3.0)}, str(f2))
    m = _two_param_model()
    assert load_pretrained(m, f1).ok and float(m.a[0, 0]) == 2.0
    m = _two_param_model()
    rep = load_pretrained(m, [f1, f2])
    assert rep.ok and float(m.b[0]) == 3.0 and not rep.optional_missing


def test_alternative_spellings_need_one_hit(tmp_path):
    from safetensors.torch import save_file

    from phyai_b200.weights.loader import load_pretrained

    def model():
        m = nn.Module()
        m.w = nn.Parameter(torch.zeros(3), requires_grad=False)
        m.w.hf_keys = {"conv.weight": None, "conv.parametrizations.weight.original1": None}
        m.w.hf_alternatives = True
        return m

    save_file({"conv.parametrizations.weight.original1": torch.ones(3)}, str(tmp_path / "model.safetensors"))
    m = model()
    rep = load_pretrained(m, tmp_path)
    assert rep.ok and rep.optional_missing == ["conv.weight"] and float(m.w[0]) == 1.0
    other = tmp_path / "empty"
    other.mkdir()
    save_file({"unrelated": torch.ones(1)}, str(other / "model.safetensors"))
    with pytest.raises(RuntimeError):
        load_pretrained(model(), other, remap=lambda k: None if k == "unrelated" else k)
