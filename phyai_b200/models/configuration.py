"""Frozen-dataclass base for model configs read from ``config.json``.

Behaviour contract (reference: phyai/src/phyai/models/configuration.py:76-171):
``from_dict`` drops unknown keys, builds nested sub-configs from nested dicts,
can pull a field from a dotted path of the source dict (``nested_sources``), and
instances read like mappings (``cfg["hidden_size"]``, ``"x" in cfg``, ``cfg.get``).
"""

from __future__ import annotations

import dataclasses
import json
import typing
from dataclasses import dataclass
from pathlib import Path
from typing import Any, ClassVar, Iterator, Mapping


def _dig(src: Mapping[str, Any], dotted: str) -> tuple[bool, Any]:
    cur: Any = src
    for part in dotted.split("."):
        if not isinstance(cur, Mapping) or part not in cur:
            return False, None
        cur = cur[part]
    return True, cur


@dataclass(frozen=True)
class PretrainedConfig:
    #: field name -> dotted path in the source dict, tried when the field itself is absent
    nested_sources: ClassVar[dict[str, str]] = {}

    # -------------------------------------------------------------- loading
    @classmethod
    def from_dict(cls, src: Mapping[str, Any]) -> "PretrainedConfig":
        hints = typing.get_type_hints(cls)
        kwargs: dict[str, Any] = {}
        for f in dataclasses.fields(cls):
            if not f.init:
                continue
            found, val = (True, src[f.name]) if f.name in src else (False, None)
            if not found and f.name in cls.nested_sources:
                found, val = _dig(src, cls.nested_sources[f.name])
            if not found:
                continue
            ftype = hints.get(f.name)
            sub = _config_type(ftype)
            if sub is not None and isinstance(val, Mapping):
                val = sub.from_dict(val)
            elif isinstance(val, list) and _wants_tuple(ftype):
                val = tuple(val)
            kwargs[f.name] = val
        return cls(**kwargs)

    @classmethod
    def from_json(cls, path: str | Path) -> "PretrainedConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            out[f.name] = v.to_dict() if isinstance(v, PretrainedConfig) else (list(v) if isinstance(v, tuple) else v)
        return out

    def to_json(self, path: str | Path) -> None:
        Path(path).write_text(json.dumps(self.to_dict(), indent=2, default=str))

    def replace(self, **changes: Any) -> "PretrainedConfig":
        return dataclasses.replace(self, **changes)

    # ------------------------------------------------------- mapping access
    def __getitem__(self, key: str) -> Any:
        if key not in self:
            raise KeyError(key)
        return getattr(self, key)

    def __contains__(self, key: object) -> bool:
        return isinstance(key, str) and any(f.name == key for f in dataclasses.fields(self))

    def __iter__(self) -> Iterator[str]:
        return (f.name for f in dataclasses.fields(self))

    def keys(self):
        return list(iter(self))

    def get(self, key: str, default: Any = None) -> Any:
        return getattr(self, key) if key in self else default


def _config_type(tp: Any) -> type | None:
    """The PretrainedConfig subclass inside ``tp`` (handles ``X | None``), if any."""
    if isinstance(tp, type) and issubclass(tp, PretrainedConfig):
        return tp
    for arg in typing.get_args(tp) or ():
        if isinstance(arg, type) and issubclass(arg, PretrainedConfig):
            return arg
    return None


def _wants_tuple(tp: Any) -> bool:
    origin = typing.get_origin(tp)
    if origin is tuple:
        return True
    return any(typing.get_origin(a) is tuple for a in (typing.get_args(tp) or ()))


__all__ = ["PretrainedConfig"]
