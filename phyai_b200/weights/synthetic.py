"""Write a random-init checkpoint with the exact key set a model expects.

The serving entries refuse to run without a checkpoint directory for some models;
benchmarks and tests use random weights, so this module turns a constructed
model into ``config.json`` + ``model.safetensors`` in the on-disk layout the
loader reads (including sharded variants with an index file).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch

from .loader import build_index


def synthetic_state_dict(model: torch.nn.Module, *, seed: int = 0, std: float = 0.02,
                         full_shapes: Mapping[str, tuple[int, ...]] | None = None) -> dict[str, torch.Tensor]:
    """One random tensor per checkpoint key. Fused parameters get one tensor per leg.

    Shapes are taken from ``param.hf_shapes[key]`` when a layer declares them (legs of
    fused or sharded parameters), else from the parameter itself.
    """
    g = torch.Generator().manual_seed(seed)
    index, _ = build_index(model)
    out: dict[str, torch.Tensor] = {}
    for key, (p, sid, _) in index.items():
        shape = None
        if full_shapes and key in full_shapes:
            shape = tuple(full_shapes[key])
        elif getattr(p, "hf_shapes", None) and key in p.hf_shapes:
            shape = tuple(p.hf_shapes[key])
        else:
            shape = tuple(p.shape)
        dt = p.dtype if p.dtype.is_floating_point and p.dtype.itemsize > 1 else torch.float32
        if key.endswith("norm.weight") or ".layernorm.weight" in key or key.endswith("_layernorm.weight"):
            t = torch.zeros(shape) + (0.0 if "gemma" in type(model).__name__.lower() else 1.0)
        else:
            t = torch.randn(shape, generator=g) * std
        out[key] = t.to(dt).contiguous()
    return out


def write_checkpoint(directory: str | Path, state: Mapping[str, torch.Tensor], config: Mapping | None = None, *,
                     shards: int = 1, stem: str = "model") -> Path:
    from safetensors.torch import save_file

    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    if config is not None:
        (d / "config.json").write_text(json.dumps(dict(config), indent=2, default=str))
    keys = list(state.keys())
    if shards <= 1:
        save_file({k: state[k].contiguous() for k in keys}, str(d / f"{stem}.safetensors"))
        return d
    per = (len(keys) + shards - 1) // shards
    weight_map = {}
    for i in range(shards):
        part = keys[i * per:(i + 1) * per]
        if not part:
            continue
        fname = f"{stem}-{i + 1:05d}-of-{shards:05d}.safetensors"
        save_file({k: state[k].contiguous() for k in part}, str(d / fname))
        weight_map.update({k: fname for k in part})
    (d / f"{stem}.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}, indent=2))
    return d


__all__ = ["synthetic_state_dict", "write_checkpoint"]
