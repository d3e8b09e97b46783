"""Attention layers.

* ``Attention``           no cache; padded 4-D ``(B, S, H, D)`` or ragged 3-D ``(T, H, D)`` inputs
* ``ARAttention``         paged KV (page size 1) for autoregressive / prefix language models
* ``DiffusionAttention``  same paged machinery, non-causal by default; used by action experts
                          whose query tokens attend [cached prefix | their own fresh K/V]

Backends: ``"b200"`` = the tcgen05 kernel of ``csrc/attention_tc.cu`` (``ops.attention``),
``"torch"`` = SDPA / eager. The paged layers follow a four-hook lifecycle so a captured
CUDA graph never re-plans: ``init_cuda_graph_state`` (allocate static metadata buffers),
``init_capture_metadata`` (bind them for capture), ``replay_metadata`` (copy new values
in place before a replay) and ``forward``.
Reference: phyai/src/phyai/layers/attention/{attention,ar,diffusion}/*.py.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...cache import KVCachePool
from ...engine_config import resolve_engine_defaults
from ...ops import ref
from .common import RaggedMeta, eager_attn


def _kernel_ok(backend: str, x: torch.Tensor) -> bool:
    return backend == "b200" and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 256


class Attention(nn.Module):
    def __init__(self, num_heads: int, head_dim: int, num_kv_heads: int | None = None, *, scale: float | None = None,
                 causal: bool = False, sliding_window: int | None = None, logits_soft_cap: float | None = None,
                 backend: str | None = None, backend_kwargs: dict | None = None) -> None:
        """``backend_kwargs`` is accepted for argument bundles written for the reference (its backends take workspace sizes
        and the like); the kernels here need none."""
        super().__init__()
        _, backend, _ = resolve_engine_defaults(None, backend, None)
        self.num_heads, self.head_dim = num_heads, head_dim
        self.num_kv_heads = num_kv_heads or num_heads
        if num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.scale = scale if scale is not None else head_dim ** -0.5
        self.causal, self.sliding_window, self.logits_soft_cap, self.backend = causal, sliding_window, logits_soft_cap, backend

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, meta: RaggedMeta | None = None,
                mask: torch.Tensor | None = None) -> torch.Tensor:
        plain = self.sliding_window is None and self.logits_soft_cap is None and mask is None
        # a sliding window (on a causal layer) and a logit soft cap are served by the tcgen05 kernel too; an explicit mask is not
        kern = mask is None and (self.sliding_window is None or self.causal)
        extra = dict(window=int(self.sliding_window or 0), soft_cap=float(self.logits_soft_cap or 0.0))
        if q.dim() == 3:                                   # ragged (T, H, D)
            if meta is None:
                raise ValueError("ragged attention needs RaggedMeta")
            cu = meta.cu_seqlens.to(torch.int32)
            start, lens = cu[:-1].contiguous(), (cu[1:] - cu[:-1]).contiguous()
            if kern and _kernel_ok(self.backend, q):
                return ops.attention(q, k, v, None, start, lens, start, lens, max_q_len=meta.max_len,
                                     causal=self.causal, sm_scale=self.scale, **extra)
            if not plain:
                if mask is not None:
                    raise NotImplementedError("ragged attention takes no explicit mask")
                # window / soft cap off the kernel path: one sequence at a time through the eager statement
                outs = [self._eager(q[s:s + n][None], k[s:s + n][None], v[s:s + n][None], None)[0]
                        for s, n in zip(start.tolist(), lens.tolist())]
                return torch.cat(outs)
            return ref.attention(q, k, v, start, lens, start, lens, causal=self.causal, sm_scale=self.scale)
        B, Sq, Hq, D = q.shape
        Sk = k.shape[1]
        if kern and _kernel_ok(self.backend, q) and q.is_contiguous() and k.is_contiguous() and v.is_contiguous():
            ar = torch.arange(B, device=q.device, dtype=torch.int32)
            out = ops.attention(q.view(B * Sq, Hq, D), k.view(B * Sk, -1, D), v.view(B * Sk, -1, D), None, ar * Sq,
                                torch.full_like(ar, Sq), ar * Sk, torch.full_like(ar, Sk), max_q_len=Sq,
                                causal=self.causal, sm_scale=self.scale, **extra)
            return out.view(B, Sq, Hq, D)
        if plain and self.backend == "torch" and q.device.type != "cpu":
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               is_causal=self.causal and Sq == Sk, scale=self.scale,
                                               enable_gqa=self.num_kv_heads != self.num_heads)
            return o.transpose(1, 2)
        return self._eager(q, k, v, mask)

    def _eager(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None) -> torch.Tensor:
        """(B, S, H, D) statement in PyTorch with every option (mask, window, soft cap)."""
        Sq, Sk = q.shape[1], k.shape[1]
        m = mask
        if self.sliding_window is not None:
            qi = torch.arange(Sq, device=q.device)[:, None] + (Sk - Sq)
            sw = (qi - torch.arange(Sk, device=q.device)[None, :]) < self.sliding_window
            m = sw if m is None else (m & sw)
        return eager_attn(q, k, v, scale=self.scale, mask=m, causal=self.causal, logits_soft_cap=self.logits_soft_cap)


@dataclass
class PagedAttnMetadata:
    """Static-shape description of one paged attention call.

    cu_seqlens_q      (B+1,) int32   query token ranges
    paged_kv_indptr   (B+1,) int32   ranges into paged_kv_indices
    paged_kv_indices  (N,)   int32   pool slot of every KV entry (page size 1)
    paged_kv_last_page_len (B,) int32  always 1 at page size 1 (kept for interface parity)
    write_indices     (T,)   int64   pool slot each new token's K/V is written to
    position_ids      (T,)   int32
    """

    cu_seqlens_q: torch.Tensor
    paged_kv_indptr: torch.Tensor
    paged_kv_indices: torch.Tensor
    write_indices: torch.Tensor
    position_ids: torch.Tensor | None = None
    paged_kv_last_page_len: torch.Tensor | None = None
    max_q_len: int = 0

    def copy_(self, other: "PagedAttnMetadata") -> None:
        for name in ("cu_seqlens_q", "paged_kv_indptr", "write_indices", "position_ids", "paged_kv_last_page_len"):
            dst, src = getattr(self, name), getattr(other, name)
            if dst is not None and src is not None:
                dst[: src.numel()].copy_(src)
        self.paged_kv_indices[: other.paged_kv_indices.numel()].copy_(other.paged_kv_indices)
        self.max_q_len = max(self.max_q_len, other.max_q_len)


ARAttnMetadata = PagedAttnMetadata
DiffusionAttnMetadata = PagedAttnMetadata


@dataclass
class PagedAttnCtx:
    kv_pool: KVCachePool
    metadata: PagedAttnMetadata


ARAttnCtx = PagedAttnCtx
DiffusionAttnCtx = PagedAttnCtx


class _PagedAttention(nn.Module):
    default_causal = True

    def __init__(self, layer_id: int, num_heads: int, head_dim: int, num_kv_heads: int | None = None, *,
                 scale: float | None = None, causal: bool | None = None, backend: str | None = None,
                 backend_kwargs: dict | None = None) -> None:
        super().__init__()
        _, backend, _ = resolve_engine_defaults(None, backend, None)
        self.layer_id, self.num_heads, self.head_dim = layer_id, num_heads, head_dim
        self.num_kv_heads = num_kv_heads or num_heads
        self.scale = scale if scale is not None else head_dim ** -0.5
        self.causal = self.default_causal if causal is None else causal
        self.backend = backend
        self._static: PagedAttnMetadata | None = None

    # ---- graph lifecycle
    def init_cuda_graph_state(self, max_tokens: int, max_batch: int, max_kv_entries: int, device) -> PagedAttnMetadata:
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=device)  # noqa: E731
        self._static = PagedAttnMetadata(z(max_batch + 1, torch.int32), z(max_batch + 1, torch.int32),
                                         z(max_kv_entries, torch.int32), z(max_tokens, torch.int64),
                                         z(max_tokens, torch.int32), z(max_batch, torch.int32))
        return self._static

    def init_capture_metadata(self, meta: PagedAttnMetadata) -> PagedAttnMetadata:
        if self._static is None:
            raise RuntimeError("init_cuda_graph_state must run before capture")
        self._static.copy_(meta)
        return self._static

    def replay_metadata(self, meta: PagedAttnMetadata) -> None:
        if self._static is None:
            raise RuntimeError("no captured metadata to refresh")
        self._static.copy_(meta)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ctx: PagedAttnCtx) -> torch.Tensor:
        """q (T, Hq, D), k/v (T, Hkv, D): write K/V to the pool, then attend over the paged entries."""
        md, pool = ctx.metadata, ctx.kv_pool
        pool.write_kv(self.layer_id, k, v, md.write_indices[: k.shape[0]])
        kp, vp = pool.layer(self.layer_id)
        cu = md.cu_seqlens_q
        q_start, q_len = cu[:-1].contiguous(), (cu[1:] - cu[:-1]).contiguous()
        kv_ptr = md.paged_kv_indptr[:-1].contiguous()
        kv_len = (md.paged_kv_indptr[1:] - md.paged_kv_indptr[:-1]).contiguous()
        if _kernel_ok(self.backend, q):
            return ops.attention(q, kp, vp, None, q_start, q_len, kv_ptr, kv_len, kv_indices=md.paged_kv_indices,
                                 max_q_len=md.max_q_len or q.shape[0], causal=self.causal, sm_scale=self.scale)
        return ref.attention(q, kp, vp, q_start, q_len, kv_ptr, kv_len, kv_indices=md.paged_kv_indices,
                             causal=self.causal, sm_scale=self.scale)


class ARAttention(_PagedAttention):
    default_causal = True


class DiffusionAttention(_PagedAttention):
    default_causal = False


__all__ = ["Attention", "ARAttention", "DiffusionAttention", "PagedAttnMetadata", "PagedAttnCtx", "ARAttnMetadata",
           "ARAttnCtx", "DiffusionAttnMetadata", "DiffusionAttnCtx"]
