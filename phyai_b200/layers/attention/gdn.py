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

from dataclasses import dataclass

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


@dataclass
class GatedDeltaNetCtx:
    """Where the recurrent state of a call lives: ``state_pool`` (slots, value heads, Dv, Dk) fp32 and one slot index per
    sequence (read as the initial state, written back with the final one); ``cu_seqlens`` for token-major inputs."""

    state_pool: torch.Tensor | None = None
    state_indices: torch.Tensor | None = None
    cu_seqlens: torch.Tensor | None = None


GDN_BACKENDS = ("chunked", "recurrent")
_BACKEND_ALIASES = {"flashinfer": "chunked", "fla": "chunked"}      # the names the reference's configurations carry


def list_gdn_backends() -> list[str]:
    return list(GDN_BACKENDS)


class GatedDeltaNet(nn.Module):
    """Gated delta rule with the gates built inside, in the reference's calling convention
    (phyai/src/phyai/layers/attention/gdn/layer.py:33-140): ``forward(q, k, v, a, b, a_log, dt_bias)`` with
    ``g = -exp(a_log) * softplus(a + dt_bias)``, ``beta = sigmoid(b)``, q / k scaled to unit length
    (``x * rsqrt(sum x^2 + 1e-6)``) and value heads a multiple of the query / key heads (each query head serves a group
    of value heads). Inputs are padded ``(B, T, H, D)`` or token-major ``(T, H, D)`` with ``cu_seqlens``; states are
    ``(sequences, value heads, Dv, Dk)``. One token per sequence with a state pool takes the decode kernel."""

    def __init__(self, num_query_heads: int, head_dim: int, *, num_key_heads: int | None = None, num_value_heads: int | None = None,
                 scale: float | None = None, use_qk_l2norm: bool = True, backend: str = "chunked", backend_kwargs: dict | None = None) -> None:
        super().__init__()
        num_key_heads = num_query_heads if num_key_heads is None else num_key_heads
        num_value_heads = num_query_heads if num_value_heads is None else num_value_heads
        if min(num_query_heads, num_key_heads, num_value_heads, head_dim) <= 0:
            raise ValueError("GatedDeltaNet: head counts and head_dim must be positive")
        if num_query_heads != num_key_heads:
            raise ValueError(f"GatedDeltaNet needs as many key heads as query heads, got {num_key_heads} and {num_query_heads}")
        if num_value_heads % num_query_heads:
            raise ValueError(f"num_value_heads={num_value_heads} must be a multiple of num_query_heads={num_query_heads}")
        name = _BACKEND_ALIASES.get(backend, backend)
        if name not in GDN_BACKENDS:
            raise KeyError(f"unknown gated-delta-net backend {backend!r}; available: {list(GDN_BACKENDS)}")
        self.num_query_heads, self.num_key_heads, self.num_value_heads = int(num_query_heads), int(num_key_heads), int(num_value_heads)
        self.num_state_heads, self.head_dim = self.num_value_heads, int(head_dim)
        self.scale = scale if scale is not None else head_dim ** -0.5
        self.use_qk_l2norm, self.backend, self.chunk = bool(use_qk_l2norm), name, int((backend_kwargs or {}).get("chunk", 64))
        self._op = GatedDeltaNetAttention(self.num_value_heads, self.head_dim, self.head_dim, backend=name)

    def extra_repr(self) -> str:
        return (f"num_query_heads={self.num_query_heads}, num_value_heads={self.num_value_heads}, head_dim={self.head_dim}, "
                f"backend={self.backend!r}")

    def _prepare(self, q, k, a, b, a_log, dt_bias):
        rep = self.num_value_heads // self.num_query_heads
        qf, kf = q.float().repeat_interleave(rep, dim=-2), k.float().repeat_interleave(rep, dim=-2)
        if self.use_qk_l2norm:
            qf = qf * torch.rsqrt(qf.square().sum(-1, keepdim=True) + 1e-6)
            kf = kf * torch.rsqrt(kf.square().sum(-1, keepdim=True) + 1e-6)
        g = -a_log.float().exp() * F.softplus(a.float() + dt_bias.float())
        return qf, kf, g, b.float().sigmoid()

    def forward(self, q, k, v, a, b, a_log, dt_bias, ctx: GatedDeltaNetCtx | None = None, *, cu_seqlens: torch.Tensor | None = None,
                initial_state: torch.Tensor | None = None, return_state: bool = False):
        if q.shape[-2] != self.num_query_heads or v.shape[-2] != self.num_value_heads or q.shape[-1] != self.head_dim:
            raise ValueError(f"GatedDeltaNet: q {tuple(q.shape)} / v {tuple(v.shape)} do not fit {self.extra_repr()}")
        ctx = ctx or GatedDeltaNetCtx(cu_seqlens=cu_seqlens)
        cu = ctx.cu_seqlens if ctx.cu_seqlens is not None else cu_seqlens
        pool, idx = ctx.state_pool, ctx.state_indices
        if pool is not None and idx is not None and initial_state is None:
            initial_state = pool[idx]
        qf, kf, g, beta = self._prepare(q, k, a, b, a_log, dt_bias)
        ragged = q.dim() == 3
        if ragged and cu is None:
            raise ValueError("token-major inputs need cu_seqlens")
        spans = list(zip(cu.tolist()[:-1], cu.tolist()[1:])) if ragged else [(None, None)] * 1
        rule = gated_delta_rule_recurrent if self.backend == "recurrent" else gated_delta_rule_chunked
        kw = dict(scale=self.scale, use_qk_l2norm=False) | ({} if self.backend == "recurrent" else {"chunk": self.chunk})
        if ragged:
            outs, finals = [], []
            for i, (s0, s1) in enumerate(spans):
                st = None if initial_state is None else initial_state[i:i + 1].transpose(-1, -2)
                o, S = rule(qf[None, s0:s1], kf[None, s0:s1], v[None, s0:s1], g[None, s0:s1], beta[None, s0:s1], st, **kw)
                outs.append(o[0])
                finals.append(S)
            out, final = torch.cat(outs), torch.cat(finals)
        else:
            st = None if initial_state is None else initial_state.transpose(-1, -2)
            out, final = rule(qf, kf, v, g, beta, st, **kw)
        final = final.transpose(-1, -2)                      # (sequences, value heads, Dv, Dk)
        if pool is not None and idx is not None:
            pool[idx] = final.to(pool.dtype)
        return (out, final) if return_state else out


__all__ = ["GatedDeltaNet", "GatedDeltaNetCtx", "GDN_BACKENDS", "list_gdn_backends", "GatedDeltaNetAttention", "gated_delta_rule_recurrent", "gated_delta_rule_chunked"]
