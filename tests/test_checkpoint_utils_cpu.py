"""Checkpoint folder resolution: local directories, hub ids through a stand-in for the download, shard discovery with
and without an index, config loading with defaults, and the CUDA helpers that must work without a GPU."""

import json
import sys
import types

import pytest
import torch

from phyai_b200.utils import checkpoint as ck


def test_local_directory_is_returned_and_a_file_is_refused(tmp_path):
    assert ck.resolve_checkpoint(tmp_path) == tmp_path
    assert ck.resolve_checkpoint(str(tmp_path)) == tmp_path
    f = tmp_path / "model.safetensors"
    f.write_bytes(b"")
    with pytest.raises(ValueError, match="is a file"):
        ck.resolve_checkpoint(f)


def test_anything_else_is_a_hub_id_forwarded_to_the_download(tmp_path, monkeypatch):
    seen = {}

    def fake_download(repo_id, revision=None, cache_dir=None):
        seen.update(repo_id=repo_id, revision=revision, cache_dir=cache_dir)
        return str(tmp_path)

    monkeypatch.setitem(sys.modules, "huggingface_hub", types.SimpleNamespace(snapshot_download=fake_download))
    got = ck.resolve_checkpoint("org/some-model", revision="v2", cache_dir="/cache")
    assert got == tmp_path and seen == {"repo_id": "org/some-model", "revision": "v2", "cache_dir": "/cache"}


def test_shard_discovery(tmp_path):
    with pytest.raises(FileNotFoundError, match="no .safetensors"):
        ck.find_safetensors(tmp_path)
    for name in ("b.safetensors", "a.safetensors"):
        (tmp_path / name).write_bytes(b"")
    assert [p.name for p in ck.find_safetensors(tmp_path)] == ["a.safetensors", "b.safetensors"]     # sorted fallback
    (tmp_path / "model.safetensors").write_bytes(b"")
    assert [p.name for p in ck.find_safetensors(tmp_path)] == ["model.safetensors"]                  # the stem wins
    (tmp_path / "vae.safetensors").write_bytes(b"")
    assert [p.name for p in ck.find_safetensors(tmp_path, stem="vae")] == ["vae.safetensors"]
    index = {"weight_map": {"w1": "b.safetensors", "w2": "a.safetensors", "w3": "b.safetensors"}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    assert [p.name for p in ck.find_safetensors(tmp_path)] == ["b.safetensors", "a.safetensors"]     # index order, once each
    index["weight_map"]["w4"] = "gone.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(FileNotFoundError, match=r"missing shards: \['gone.safetensors'\]"):
        ck.find_safetensors(tmp_path)


def test_load_config_reads_json_or_falls_back_to_defaults(tmp_path):
    from phyai_b200.models.pi05 import PI05Config

    assert ck.load_config(tmp_path, PI05Config) == PI05Config()
    (tmp_path / "config.json").write_text(json.dumps({"chunk_size": 25, "no_such_field": 1}))
    cfg = ck.load_config(tmp_path, PI05Config)
    assert cfg.chunk_size == 25 and not hasattr(cfg, "no_such_field")


def test_cuda_helpers_without_a_gpu(monkeypatch, caplog):
    from phyai_b200.utils import cuda as cu

    monkeypatch.setenv("LOCAL_RANK", "3")
    assert cu.local_rank() == 3
    monkeypatch.delenv("LOCAL_RANK")
    assert cu.local_rank() == 0
    dev = cu.init_cuda("cpu", torch.float32)
    assert dev.type == "cpu"
    cu.init_cublas()                                  # nothing to initialise: the GEMMs are this package's own
    if not torch.cuda.is_available():
        assert cu.sm_arch() == 0 and cu.topology_lines() == ["no CUDA device visible"]
        with caplog.at_level("INFO"):
            cu.print_topology()
            cu.print_distributed_topology()          # no process group: this rank's own line
        text = " ".join(r.getMessage() for r in caplog.records)
        assert "no CUDA device visible" in text and "rank 0 on" in text
