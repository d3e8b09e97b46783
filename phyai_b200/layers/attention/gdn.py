"""Gated DeltaNet linear attention (Qwen3.5-style hybrid layers).

State per head ``S`` (Dk x Dv). Per token: ``S <- exp(g_t) * S``; ``v_new = (v_t - S^T k_t) * beta_t``;
``S <- S + k_t v_new^T``; ``o_t = S^T q_t``.

Three evaluations of the same rule:

* :func:`gated_delta_rule_recurrent`  token by token, the oracle;
* :func:`gated_delta_rule_chunked`    prefill in chunks of 64 tokens: inside a chunk the rule is a unit lower
  triangular system ``(I + A) U = beta * (V - gamma * K S_0)`` with ``A[j, l] = beta_j gamma_j / gamma_l (k_j . k_l)``
  (``gamma`` = running decay since the chunk start), solved once per chunk; outputs and the next state are
  matrix products. ``T / 64`` sequential steps of batched GEMMs instead of ``T`` steps of rank-1 updates;
* ``ops.gdn_decode``                  one token per sequence against a state pool, one kernel (``csrc/gdn.cu``).

Reference: phyai/src/phyai/layers/attention/gdn/{layer,base}.py and backends/{fla,flashinfer}.py (chunked
prefill backends/flashinfer.py:113-160, recurrent decode :161-208).
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


def gated_delta_rule_chunked(q, k, v, g, beta, state=None, *, scale: float | None = None, use_qk_l2norm: bool = True,
                             chunk: int = 64):
    """Same contract as :func:`gated_delta_rule_recurrent`, evaluated chunk-wise (fp32 inside)."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    qf, kf, vf = q.float(), k.float(), v.float()
    if use_qk_l2norm:
        qf, kf = F.normalize(qf, dim=-1), F.normalize(kf, dim=-1)
    qf = qf * (Dk ** -0.5 if scale is None else scale)
    gf, bf = g.float(), beta.float()
    pad = (-T) % chunk
    if pad:   # padded tokens: beta = 0 and g = 0 leave the state alone; their outputs are dropped
        qf, kf, vf = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (qf, kf, vf))
        gf, bf = F.pad(gf, (0, 0, 0, pad)), F.pad(bf, (0, 0, 0, pad))
    n = (T + pad) // chunk
    # (B, H, n, C, D) views
    def split(t):
        return t.reshape(B, n, chunk, H, -1).permute(0, 3, 1, 2, 4)
    qc, kc, vc = split(qf), split(kf), split(vf)
    gc = gf.reshape(B, n, chunk, H).permute(0, 3, 1, 2)
    bc = bf.reshape(B, n, chunk, H).permute(0, 3, 1, 2)
    G = gc.cumsum(-1)                                              # log decay since the chunk start, inclusive
    ratio = (G[..., :, None] - G[..., None, :]).tril().exp().tril()  # gamma_i / gamma_j for j <= i, 0 above the diagonal
    kk = kc @ kc.transpose(-1, -2)
    A = (bc[..., :, None] * ratio * kk).tril(-1)
    eye = torch.eye(chunk, device=q.device, dtype=torch.float32)
    # T = (I + A)^-1 applied to [beta V | beta gamma K] in one triangular solve per chunk
    rhs = torch.cat([bc[..., None] * vc, (bc * G.exp())[..., None] * kc], dim=-1)
    sol = torch.linalg.solve_triangular(eye + A, rhs, upper=False, unitriangular=True)
    TV, TK = sol[..., :Dv], sol[..., Dv:]                          # (B,H,n,C,Dv), (B,H,n,C,Dk)
    qk = (qc @ kc.transpose(-1, -2)) * ratio                       # (q_i . k_j) gamma_i / gamma_j, j <= i
    gam = G.exp()
    gam_end = gam[..., -1]
    S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=q.device) if state is None else state.float().clone()
    out = torch.empty(B, H, n, chunk, Dv, dtype=torch.float32, device=q.device)
    kdec = kc * (gam_end[..., None] / gam)[..., None]              # k_j gamma_C / gamma_j
    for c in range(n):
        U = TV[:, :, c] - TK[:, :, c] @ S                          # new values of the chunk
        out[:, :, c] = gam[:, :, c][..., None] * (qc[:, :, c] @ S) + qk[:, :, c] @ U
        S = gam_end[:, :, c][..., None, None] * S + kdec[:, :, c].transpose(-1, -2) @ U
    o = out.permute(0, 2, 3, 1, 4).reshape(B, n * chunk, H, Dv)[:, :T]
    return o.to(v.dtype), S


class GatedDeltaNetAttention(nn.Module):
    """Stateless op wrapper: the caller owns projections; this layer owns the state pool plumbing."""

    def __init__(self, num_heads: int, head_k_dim: int, head_v_dim: int, *, backend: str | None = None) -> None:
        super().__init__()
        self.num_heads, self.head_k_dim, self.head_v_dim = num_heads, head_k_dim, head_v_dim
        self.backend = backend or "chunked"      # "chunked" | "recurrent" (the token-by-token oracle)
        self.chunk = 64

    def prefill(self, q, k, v, g, beta, *, state_pool: torch.Tensor | None = None,
                state_indices: torch.Tensor | None = None):
        init = state_pool[state_indices] if state_pool is not None and state_indices is not None else None
        if self.backend == "recurrent" or q.shape[1] < 2:
            o, S = gated_delta_rule_recurrent(q, k, v, g, beta, init)
        else:
            o, S = gated_delta_rule_chunked(q, k, v, g, beta, init, chunk=self.chunk)
        if state_pool is not None and state_indices is not None:
            state_pool[state_indices] = S.to(state_pool.dtype)
        return o

    def decode(self, q, k, v, g, beta, *, state_pool: torch.Tensor, state_indices: torch.Tensor):
        """One token per sequence: q,k (B,H,Dk), v (B,H,Dv), g,beta (B,H). On CUDA with an fp32 pool this is one
        launch of ``gdn_decode_kernel`` that updates the pool rows in place; elsewhere the recurrence in PyTorch."""
        from ... import ops

        if (q.is_cuda and state_pool.dtype == torch.float32 and state_pool.is_contiguous() and ops.available()
                and self.head_k_dim <= 256 and self.head_v_dim % 4 == 0):
            return ops.gdn_decode(q, k, v, g, beta, state_pool, state_indices)
        o, S = gated_delta_rule_recurrent(q[:, None], k[:, None], v[:, None], g[:, None], beta[:, None],
                                          state_pool[state_indices])
        state_pool[state_indices] = S.to(state_pool.dtype)
        return o[:, 0]

    forward = prefill


__all__ = ["GatedDeltaNetAttention", "gated_delta_rule_recurrent", "gated_delta_rule_chunked"]
