"""Vocabulary-parallel embedding and LM head.

The vocabulary is padded to a multiple of ``tp * 64`` and split by rows over the ``tp``
axis. A lookup maps ids outside this rank's range to zero rows (the masked-embedding
kernel on CUDA, an index + mask in PyTorch elsewhere) and an all-reduce over ``tp``
completes it. ``ParallelLMHead`` projects hidden states to the local vocabulary slice,
optionally gathering the slices. Reference: phyai/src/phyai/layers/vocab_embedding/{layers,ops}.py.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .. import parallel as P
from ..engine_config import get_engine_config
from ..ops import ref
from ..parallel import state as pstate
from ..weights import shards

PAD_MULTIPLE = 64


def pad_vocab(vocab: int, tp: int, multiple: int = PAD_MULTIPLE) -> int:
    """``vocab`` rounded up to a multiple of ``tp * multiple``: equal shards whose rows are a multiple of ``multiple``."""
    if tp <= 0 or multiple <= 0:
        raise ValueError(f"pad_vocab: tp and multiple must be positive, got {tp} and {multiple}")
    m = tp * multiple
    return (vocab + m - 1) // m * m


def masked_embedding_lookup(ids: torch.Tensor, table: torch.Tensor, lo: int, hi: int, scale: float = 1.0) -> torch.Tensor:
    """``table[id - lo] * scale`` for ``lo <= id < hi``, zero rows otherwise."""
    flat = ids.reshape(-1).contiguous()
    if table.is_cuda and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0 and flat.dtype == torch.int64:
        out = torch.empty(flat.numel(), table.shape[1], dtype=table.dtype, device=table.device)
        ops.embedding(flat, table, out, lo=lo, hi=hi, scale=scale)
        return out.reshape(*ids.shape, -1)
    return ref.embedding(ids, table, lo, hi, scale)


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, *, params_dtype: torch.dtype | None = None,
                 embed_scale: float | None = None, axis: str = "tp", mesh=None, device=None, prefix: str = "",
                 padding_multiple: int = PAD_MULTIPLE) -> None:
        super().__init__()
        cfg = get_engine_config()
        m = mesh if mesh is not None else pstate.default_mesh()
        self.axis, self.mesh = axis, m
        self.tp_rank = m.axis_local_rank(axis) if m is not None else 0
        self.tp_size = m.axis_size(axis) if m is not None else 1
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padded = pad_vocab(num_embeddings, self.tp_size, padding_multiple)
        self.per_rank = self.padded // self.tp_size
        self.lo, self.hi = self.tp_rank * self.per_rank, (self.tp_rank + 1) * self.per_rank
        self.embed_scale = 1.0 if embed_scale is None else float(embed_scale)
        self.weight = nn.Parameter(torch.zeros(self.per_rank, embedding_dim, dtype=params_dtype or cfg.device.params_dtype,
                                               device=device if device is not None else cfg.device.target),
                                   requires_grad=False)
        if prefix:
            self.weight.hf_keys = {f"{prefix}.weight": None}
            self.weight.hf_shapes = {f"{prefix}.weight": (num_embeddings, embedding_dim)}
        self.weight.weight_loader = shards.vocab(self.padded, axis, mesh)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        y = masked_embedding_lookup(input_ids, self.weight, self.lo, self.hi, self.embed_scale)
        if self.tp_size > 1:
            y = P.all_reduce(y, axis=self.axis, mesh=self.mesh)
        return y


class ParallelLMHead(nn.Module):
    """Logits over the local vocabulary slice; ``tied`` shares the embedding's weight."""

    def __init__(self, embedding: VocabParallelEmbedding | None = None, *, num_embeddings: int | None = None,
                 embedding_dim: int | None = None, gather_output: bool = True, **kw) -> None:
        super().__init__()
        self.embedding = embedding if embedding is not None else VocabParallelEmbedding(num_embeddings, embedding_dim, **kw)
        self.gather_output = gather_output

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        e = self.embedding
        logits = F.linear(hidden, e.weight)
        if e.tp_size > 1 and self.gather_output:
            logits = P.all_gather(logits, axis=e.axis, dim=-1, mesh=e.mesh)
        return logits[..., : e.num_embeddings] if (e.tp_size == 1 or self.gather_output) else logits


pad_vocab_to = pad_vocab

__all__ = ["VocabParallelEmbedding", "ParallelLMHead", "masked_embedding_lookup", "pad_vocab", "pad_vocab_to"]
