"""Tokenizer loading (``transformers.AutoTokenizer``) with a tiny offline stand-in for tests.

Reference: phyai-utils-tools/src/phyai_utils_tools/tokenizer/loader.py:25-64.
"""

from __future__ import annotations

import functools
from typing import Any

import torch


@functools.lru_cache(maxsize=8)
def get_tokenizer(name_or_path: str, *, use_fast: bool = True, **kw: Any):
    """A local directory or a hub id (the latter needs network access or a warm cache)."""
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(name_or_path, use_fast=use_fast, **kw)


class ByteTokenizer:
    """UTF-8 bytes + 3 as ids (0 pad, 1 bos, 2 eos). For tests and synthetic benchmarks only: no vocabulary file needed."""

    pad_token_id, bos_token_id, eos_token_id = 0, 1, 2
    accepts_padding_side = True

    def __init__(self, add_bos: bool = True) -> None:
        self.add_bos = add_bos

    def __call__(self, texts, max_length: int = 64, padding: str = "max_length", truncation: bool = True,
                 return_tensors: str = "pt", padding_side: str = "right"):
        rows = []
        for s in texts:
            ids = ([self.bos_token_id] if self.add_bos else []) + [b + 3 for b in s.encode("utf-8")]
            rows.append(ids[:max_length] if truncation else ids)
        width = max_length if padding == "max_length" else max(len(r) for r in rows)
        ids = torch.zeros(len(rows), width, dtype=torch.long)
        mask = torch.zeros(len(rows), width, dtype=torch.long)
        for i, r in enumerate(rows):
            sl = slice(0, len(r)) if padding_side == "right" else slice(width - len(r), width)
            ids[i, sl] = torch.tensor(r, dtype=torch.long)
            mask[i, sl] = 1
        return {"input_ids": ids, "attention_mask": mask}

    def decode(self, ids) -> str:
        return bytes(int(i) - 3 for i in ids if int(i) >= 3).decode("utf-8", errors="replace")


__all__ = ["get_tokenizer", "ByteTokenizer"]
