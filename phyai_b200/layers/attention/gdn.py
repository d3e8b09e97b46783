"""Gated DeltaNet linear attention (Qwen3.5-style hybrid layers).

State per head ``S`` (Dk x Dv). Per token: ``S <- exp(g_t) * S``; ``v_new = (v_t - S^T k_t) * beta_t``;
``S <- S + k_t v_new^T``; ``o_t = S^T q_t``. ``prefill`` runs the recurrence over a sequence in
chunks (exact, chunk size only bounds the Python loop granularity), ``decode`` advances one
token using cached states addressed by ``state_indices``.
Reference: phyai/src/phyai/layers/attention/gdn/{layer,base}.py and backends/{fla,flashinfer}.py.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def gated_delta_rule_recurrent(q, k, v, g, beta, state=None, *, scale: float | None = None, use_qk_l2norm: bool = True):
    """q,k (B,T,H,Dk); v (B,T,H,Dv); g,beta (B,T,H). Returns (o (B,T,H,Dv), final state (B,H,Dk,Dv))."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    qf, kf, vf = q.float(), k.float(), v.float()
    if use_qk_l2norm:
        qf, kf = F.normalize(qf, dim=-1), F.normalize(kf, dim=-1)
    scale = Dk ** -0.5 if scale is None else scale
    qf = qf * scale
    S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=q.device) if state is None else state.float().clone()
    out = torch.empty(B, T, H, Dv, dtype=torch.float32, device=q.device)
    gf, bf = g.float(), beta.float()
    for t in range(T):
        S = S * gf[:, t].exp()[..., None, None]
        kt, vt = kf[:, t], vf[:, t]
        pred = torch.einsum("bhkv,bhk->bhv", S, kt)
        vnew = (vt - pred) * bf[:, t][..., None]
        S = S + torch.einsum("bhk,bhv->bhkv", kt, vnew)
        out[:, t] = torch.einsum("bhkv,bhk->bhv", S, qf[:, t])
    return out.to(v.dtype), S


class GatedDeltaNetAttention(nn.Module):
    """Stateless op wrapper: the caller owns projections; this layer owns the state pool plumbing."""

    def __init__(self, num_heads: int, head_k_dim: int, head_v_dim: int, *, backend: str | None = None) -> None:
        super().__init__()
        self.num_heads, self.head_k_dim, self.head_v_dim = num_heads, head_k_dim, head_v_dim
        self.backend = backend or "torch"

    def prefill(self, q, k, v, g, beta, *, state_pool: torch.Tensor | None = None,
                state_indices: torch.Tensor | None = None):
        init = state_pool[state_indices] if state_pool is not None and state_indices is not None else None
        o, S = gated_delta_rule_recurrent(q, k, v, g, beta, init)
        if state_pool is not None and state_indices is not None:
            state_pool[state_indices] = S.to(state_pool.dtype)
        return o

    def decode(self, q, k, v, g, beta, *, state_pool: torch.Tensor, state_indices: torch.Tensor):
        """One token per sequence: q,k (B,H,Dk), v (B,H,Dv), g,beta (B,H)."""
        o, S = gated_delta_rule_recurrent(q[:, None], k[:, None], v[:, None], g[:, None], beta[:, None],
                                          state_pool[state_indices])
        state_pool[state_indices] = S.to(state_pool.dtype)
        return o[:, 0]

    forward = prefill


__all__ = ["GatedDeltaNetAttention", "gated_delta_rule_recurrent"]
