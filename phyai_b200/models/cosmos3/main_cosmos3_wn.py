"""Plugin ``cosmos3_wn``: Cosmos3 generation over a ``cfg x tp`` mesh.

The networks and the denoising loop are those of the single-GPU plugin; the mesh decides that the
two guidance branches run on different rank groups (``cfg``), that the transformer's projections are
sharded (``tp``) and that the VAE decodes spatial tiles in parallel. Every rank takes the same
request and returns the same result.

Reference: phyai/src/phyai/models/cosmos3/main_cosmos3_wn.py:53-189.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

from ...engine import Engine, EntryArgs
from .main_cosmos3 import Cosmos3Args, Cosmos3Entry


@dataclass
class Cosmos3WNArgs(Cosmos3Args):
    pass


@Engine.register
class Cosmos3WNEntry(Cosmos3Entry):
    name: ClassVar[str] = "cosmos3_wn"
    args_cls: ClassVar[type[EntryArgs]] = Cosmos3WNArgs


__all__ = ["Cosmos3WNArgs", "Cosmos3WNEntry"]
