"""Plugin ``cosmos3_policy_wn``: Cosmos3 action inference over a ``cfg x tp`` mesh (same request on every rank).

Reference: phyai/src/phyai/models/cosmos3/main_cosmos3_policy_wn.py:40-156.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

from ...engine import Engine, EntryArgs
from .main_cosmos3_policy import Cosmos3PolicyArgs, Cosmos3PolicyEntry


@dataclass
class Cosmos3PolicyWNArgs(Cosmos3PolicyArgs):
    pass


@Engine.register
class Cosmos3PolicyWNEntry(Cosmos3PolicyEntry):
    name: ClassVar[str] = "cosmos3_policy_wn"
    args_cls: ClassVar[type[EntryArgs]] = Cosmos3PolicyWNArgs


__all__ = ["Cosmos3PolicyWNArgs", "Cosmos3PolicyWNEntry"]
