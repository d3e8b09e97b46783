"""Checkpoint folder resolution (reference: phyai/src/phyai/utils/checkpoint.py:57-177).

A checkpoint is a HuggingFace-style folder: ``config.json`` plus either
``model.safetensors`` or ``model.safetensors.index.json`` with its shards.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Type, TypeVar

C = TypeVar("C")


def resolve_checkpoint(source: str | Path, *, revision: str | None = None, cache_dir: str | None = None) -> Path:
    """A local directory as is; anything else is treated as a hub repo id and downloaded."""
    p = Path(source).expanduser()
    if p.is_dir():
        return p
    if p.exists():
        raise ValueError(f"checkpoint source {source!r} is a file; expected a directory or a hub repo id")
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:  # pragma: no cover
        raise FileNotFoundError(f"{source!r} is not a local directory and huggingface_hub is unavailable") from e
    return Path(snapshot_download(repo_id=str(source), revision=revision, cache_dir=cache_dir))


def find_safetensors(directory: str | Path, *, stem: str = "model") -> list[Path]:
    """Shard files of a checkpoint, de-duplicated, index order first."""
    d = Path(directory)
    index = d / f"{stem}.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        seen: dict[str, None] = {}
        for fname in weight_map.values():
            seen.setdefault(fname, None)
        shards = [d / f for f in seen]
        missing = [s for s in shards if not s.is_file()]
        if missing:
            raise FileNotFoundError(f"index {index} names missing shards: {[m.name for m in missing]}")
        return shards
    single = d / f"{stem}.safetensors"
    if single.is_file():
        return [single]
    found = sorted(d.glob("*.safetensors"))
    if not found:
        raise FileNotFoundError(f"no .safetensors files under {d}")
    return found


def load_config(directory: str | Path, config_cls: Type[C], *, filename: str = "config.json") -> C:
    """Read ``config.json`` into ``config_cls`` (unknown keys dropped); defaults if the file is absent."""
    f = resolve_checkpoint(directory) / filename
    if not f.is_file():
        return config_cls()
    return config_cls.from_json(f)


__all__ = ["resolve_checkpoint", "find_safetensors", "load_config"]
