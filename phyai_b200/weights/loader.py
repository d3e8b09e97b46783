"""``load_pretrained``: stream safetensors shards into a module tree.

Parameters advertise the checkpoint keys they accept through attributes set by
the layers (reference protocol: phyai/src/phyai/weights/loader.py:174-318):

* ``param.hf_keys``      ``{checkpoint_key: shard_id}`` (or a list of keys, shard_id None)
* ``param.weight_loader`` ``loader(param, tensor, shard_id)`` (default: replicated copy)
* ``param.optional``     missing keys are reported separately and never fail ``strict``
* ``param.hf_alternatives`` the keys are alternative spellings of one tensor: at least one of them
  must be present, the others are not reported as missing

Parameters without ``hf_keys`` are looked up under their dotted module path but, as in the
reference (which skips them), never count as missing. ``remap`` is a callable (``None`` drops the
key) or a dict of ordered substring rewrites (reference loader.py:87-110); ``source`` is a
checkpoint folder, a hub repo id, one safetensors file or an iterable of files. After all shards
are consumed every module's ``post_load()`` hook runs (quantisation fan-out, packed layouts,
exponentiated Snake parameters ...).
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Iterable, Mapping

import torch

from ..utils.checkpoint import find_safetensors, resolve_checkpoint
from ..utils.logging import this_rank_log
from . import shards

logger = logging.getLogger(__name__)
Remap = Callable[[str], "str | None"] | Mapping[str, "str | None"] | None


@dataclass
class LoadReport:
    loaded: list[str] = field(default_factory=list)
    missing: list[str] = field(default_factory=list)
    optional_missing: list[str] = field(default_factory=list)
    unexpected: list[str] = field(default_factory=list)
    dropped: list[str] = field(default_factory=list)
    casts: dict[str, tuple[torch.dtype, torch.dtype]] = field(default_factory=dict)

    def summary(self) -> str:
        return (f"loaded {len(self.loaded)} tensors, missing {len(self.missing)}, "
                f"optional missing {len(self.optional_missing)}, unexpected {len(self.unexpected)}, "
                f"dropped by remap {len(self.dropped)}, dtype casts {len(self.casts)}")

    @property
    def ok(self) -> bool:
        return not self.missing and not self.unexpected


def _apply_remap(remap: Remap, key: str) -> str | None:
    if remap is None:
        return key
    if callable(remap):
        return remap(key)
    if not isinstance(remap, Mapping):
        raise TypeError(f"remap must be callable, a dict or None; got {type(remap).__name__}")
    for src, dst in remap.items():          # ordered substring rewrites; a None target drops the key
        if src in key:
            if dst is None:
                return None
            key = key.replace(src, dst)
    return key


def _resolve_source(source: "str | Path | Iterable[str | Path]", stem: str) -> tuple[list[Path], str]:
    """Shard files of ``source`` (folder / repo id / one file / iterable of files) and a label for the log."""
    if isinstance(source, (str, Path)):
        p = Path(source).expanduser()
        if p.is_file():
            return [p], p.name
        directory = resolve_checkpoint(source)
        return find_safetensors(directory, stem=stem), str(directory)
    files = [Path(f) for f in source]
    if not files:
        raise FileNotFoundError("load_pretrained: empty list of safetensors files")
    return files, "weights"


def build_index(model: torch.nn.Module) -> tuple[dict[str, tuple[torch.nn.Parameter, object, str]], set[str]]:
    """``checkpoint_key -> (param, shard_id, param_name)`` plus the set of keys whose absence is not an error
    by itself (optional parameters, parameters without ``hf_keys``, alternative spellings: for the latter
    :func:`load_pretrained` still wants one spelling per parameter)."""
    index: dict[str, tuple[torch.nn.Parameter, object, str]] = {}
    optional: set[str] = set()
    tensors: Iterable[tuple[str, torch.Tensor]] = list(model.named_parameters()) + [
        (n, b) for n, b in model.named_buffers() if getattr(b, "hf_keys", None) is not None]
    for name, p in tensors:
        keys = getattr(p, "hf_keys", None)
        if keys is None:
            table = {name: None}
        elif isinstance(keys, Mapping):
            table = dict(keys)
        else:
            table = {k: None for k in keys}
        for k, sid in table.items():
            if k in index and index[k][0] is not p:
                raise ValueError(f"checkpoint key {k!r} is claimed by both {index[k][2]!r} and {name!r}")
            index[k] = (p, sid, name)
            if keys is None or getattr(p, "optional", False) or getattr(p, "hf_alternatives", False):
                optional.add(k)
    return index, optional


def load_pretrained(model: torch.nn.Module, source: "str | Path | Iterable[str | Path]", *, remap: Remap = None,
                    strict: bool = True, stem: str = "model", progress: bool = False) -> LoadReport:
    from safetensors import safe_open

    files, directory = _resolve_source(source, stem)
    index, optional = build_index(model)
    report = LoadReport()
    seen: set[str] = set()
    iterator: Iterable[Path] = files
    if progress:
        try:
            from tqdm import tqdm

            iterator = tqdm(files, desc="loading shards")
        except ImportError:
            pass
    with torch.no_grad():
        for f in iterator:
            with safe_open(str(f), framework="pt", device="cpu") as sf:
                for raw in sf.keys():
                    key = _apply_remap(remap, raw)
                    if key is None:
                        report.dropped.append(raw)
                        continue
                    hit = index.get(key)
                    if hit is None:
                        report.unexpected.append(raw)
                        continue
                    p, sid, _ = hit
                    t = sf.get_tensor(raw)
                    if t.dtype != p.dtype and t.dtype.is_floating_point:
                        report.casts[key] = (t.dtype, p.dtype)
                    loader = getattr(p, "weight_loader", None) or shards.replicated()
                    try:
                        loader(p, t, sid)
                    except Exception as e:
                        raise type(e)(f"while loading {raw!r} -> {key!r}: {e}") from e
                    seen.add(key)
                    report.loaded.append(key)
    # alternative spellings: a parameter none of whose keys showed up is missing after all
    unmet: set[str] = set()
    by_param: dict[int, list[str]] = {}
    for k, (p, _, _) in index.items():
        if getattr(p, "hf_alternatives", False) and not getattr(p, "optional", False):
            by_param.setdefault(id(p), []).append(k)
    for ks in by_param.values():
        if not any(k in seen for k in ks):
            unmet.add(ks[0])
    for k in index:
        if k not in seen:
            (report.missing if k in unmet or k not in optional else report.optional_missing).append(k)
    this_rank_log(logger, logging.INFO, "%s: %s", directory, report.summary())
    if strict and not report.ok:
        raise RuntimeError(f"strict load failed: missing={report.missing[:8]} unexpected={report.unexpected[:8]} "
                           f"({report.summary()})")
    run_post_load(model)
    return report


def run_post_load(model: torch.nn.Module) -> None:
    for m in model.modules():
        hook = getattr(m, "post_load", None)
        if callable(hook):
            hook()


__all__ = ["LoadReport", "load_pretrained", "build_index", "run_post_load"]
