"""Forward-batch payloads handed from schedulers to runners
(reference: phyai/src/phyai/payload/*.py)."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class VisionForwardBatch:
    pixel_values: torch.Tensor            # (n_img, C, H, W)


@dataclass
class LLMForwardBatch:
    hidden_states: torch.Tensor           # (tokens, hidden) packed prefix rows
    position_ids: torch.Tensor            # (tokens,) int32
    write_indices: torch.Tensor           # (tokens,) int64 KV-pool slots


@dataclass
class ExpertForwardBatch:
    x_t: torch.Tensor                     # (B, chunk, action_dim) current sample
    time_emb: torch.Tensor | None = None  # (B, hidden) AdaRMS condition


@dataclass
class VLMForwardBatch:
    pixel_values: torch.Tensor
    input_ids: torch.Tensor
    lang_lens: torch.Tensor


__all__ = ["VisionForwardBatch", "LLMForwardBatch", "ExpertForwardBatch", "VLMForwardBatch"]
