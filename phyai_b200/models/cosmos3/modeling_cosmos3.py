"""Cosmos3 "MoT" flow-matching transformer: a causal UND text tower whose per-layer K/V are
computed once per prompt, and a GEN tower whose tokens (video patches [+ action | + sound
tokens]) attend ``[K_und | K_gen]`` non-causally. The diffusion time enters as an additive
embedding on the noised tokens (no adaLN). One checkpoint layer ``layers.{i}`` feeds both
towers (``cosmos3_weight_remap``). Tensor parallel over heads / MLP columns.

Reference: phyai/src/phyai/models/cosmos3/modeling_cosmos3.py:29-1135.

Execution. ``Cosmos3Transformer.forward`` is written against this package's layers, so on
CPU it is plain PyTorch (the oracle) and on B200 every heavy op is one of this repository's
kernels: tcgen05 GEMMs (gated activation and residual add fused in their epilogues), one
kernel for per-head q/k RMSNorm + mRoPE + K/V placement, and the tcgen05 attention kernel
reading a K/V buffer that holds the text K/V in front and receives the GEN K/V behind them
(the reference concatenates ``cat([K_und, K])`` / ``cat([V_und, V])`` in every layer of every
step, modeling_cosmos3.py:403-404).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ... import parallel as P
from ...engine_config import get_engine_config, resolve_engine_defaults
from ...layers.attention import Attention
from ...layers.layer_norm import RMSNorm
from ...layers.linear import QKVParallelLinear, ReplicatedLinear, RowParallelLinear
from ...layers.mlp import DenseMLP
from ...layers.rotary_embedding import MRotaryEmbedding
from ...layers.vocab_embedding import VocabParallelEmbedding
from ...ops import ref
from .configuration_cosmos3 import Cosmos3Config


# ----------------------------------------------------------------- positions
def compute_mrope_position_ids_text(num_tokens: int, temporal_offset: int) -> tuple[torch.Tensor, int]:
    """Text: the three axes share one increasing id."""
    ids = torch.arange(num_tokens, dtype=torch.long) + temporal_offset
    return ids[None].expand(3, -1).contiguous(), temporal_offset + num_tokens


def compute_mrope_position_ids_vision(grid_t: int, grid_h: int, grid_w: int, temporal_offset, fps: float | None = None,
                                      base_fps: float = 24.0, temporal_compression_factor: int = 4,
                                      base_temporal_compression_factor: int | None = None,
                                      enable_fps_modulation: bool = True, start_frame_offset: int = 0):
    """(t, h, w) ids of a token grid, t-major. With fps modulation the time axis is rescaled so
    clips at different frame rates share one temporal coordinate (float positions)."""
    modulated = enable_fps_modulation and fps is not None
    if modulated:
        tps = fps / temporal_compression_factor
        base_tcf = base_temporal_compression_factor if base_temporal_compression_factor is not None else temporal_compression_factor
        base_tps = base_fps / base_tcf
        t_idx = (torch.arange(grid_t, dtype=torch.float32) + start_frame_offset) / tps * base_tps + temporal_offset
    else:
        t_idx = torch.arange(grid_t, dtype=torch.long) + int(temporal_offset) + start_frame_offset
    t_index = t_idx.view(-1, 1).expand(-1, grid_h * grid_w).flatten()
    h_index = torch.arange(grid_h).view(1, -1, 1).expand(grid_t, -1, grid_w).flatten()
    w_index = torch.arange(grid_w).view(1, 1, -1).expand(grid_t, grid_h, -1).flatten()
    if modulated:
        ids = torch.stack([t_index, h_index.float(), w_index.float()])
    else:
        ids = torch.stack([t_index, h_index, w_index])
    return ids, math.floor(ids.max().item()) + 1


def local_head_counts(tp_size: int, num_attention_heads: int, num_key_value_heads: int) -> tuple[int, int]:
    if num_attention_heads % tp_size or num_key_value_heads % tp_size:
        raise ValueError(f"tp_size={tp_size} must divide both num_attention_heads={num_attention_heads} and "
                         f"num_key_value_heads={num_key_value_heads}")
    return num_attention_heads // tp_size, num_key_value_heads // tp_size


# -------------------------------------------------------------------- pieces
class TimestepEmbedder(nn.Module):
    def __init__(self, hidden_size: int, frequency_embedding_size: int = 256, max_period: int = 10000, *,
                 params_dtype=None, device=None, prefix: str = "") -> None:
        super().__init__()
        device = device if device is not None else get_engine_config().device.target
        self.linear_1 = ReplicatedLinear(frequency_embedding_size, hidden_size, bias=True, params_dtype=params_dtype,
                                         prefix=f"{prefix}.linear_1" if prefix else "")
        self.linear_2 = ReplicatedLinear(hidden_size, hidden_size, bias=True, params_dtype=params_dtype,
                                         prefix=f"{prefix}.linear_2" if prefix else "")
        half = frequency_embedding_size // 2
        freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=device) / half)
        self.register_buffer("freqs", freqs, persistent=False)

    def forward(self, t: torch.Tensor) -> torch.Tensor:
        a = t[:, None].float() * self.freqs[None]
        f = torch.cat([a.cos(), a.sin()], dim=-1).to(self.linear_1.weight.dtype)
        h, _ = self.linear_1(f)
        out, _ = self.linear_2(F.silu(h.float()).to(h.dtype))
        return out


class DomainAwareLinear(nn.Module):
    """One ``(in, out)`` weight and bias per embodiment domain; rows picked by ``domain_id``."""

    def __init__(self, input_size: int, output_size: int, num_domains: int, *, params_dtype=None, device=None,
                 prefix: str = "") -> None:
        super().__init__()
        cfg = get_engine_config()
        device = device if device is not None else cfg.device.target
        dt = params_dtype or cfg.device.params_dtype
        self.input_size, self.output_size = input_size, output_size
        self.fc = nn.Parameter(torch.zeros(num_domains, output_size * input_size, dtype=dt, device=device), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(num_domains, output_size, dtype=dt, device=device), requires_grad=False)
        if prefix:
            self.fc.hf_keys = {f"{prefix}.fc.weight": None}
            self.bias.hf_keys = {f"{prefix}.bias.weight": None}

    def forward(self, x: torch.Tensor, domain_id: torch.Tensor) -> torch.Tensor:
        b = x.shape[0]
        if x.is_cuda and x.dtype == torch.bfloat16 and self.fc.dtype == torch.bfloat16 and domain_id.is_cuda:
            # own kernel: picks each sample's weight by the domain id it reads on the device
            x3 = x[:, None] if x.dim() == 2 else x
            y = ops.domain_linear(x3.contiguous(), self.fc, self.bias, domain_id.to(torch.int64).contiguous())
            return y[:, 0] if x.dim() == 2 else y
        w = self.fc[domain_id].view(b, self.input_size, self.output_size)
        bias = self.bias[domain_id]
        if x.dim() == 2:
            return torch.bmm(x[:, None], w)[:, 0] + bias
        return torch.bmm(x, w) + bias[:, None]


class Cosmos3Attention(nn.Module):
    """q/k/v + per-head RMSNorm + mRoPE + attention + out projection, for either tower."""

    def __init__(self, cfg: Cosmos3Config, *, causal: bool, attn_backend: str, norm_backend: str, params_dtype, prefix: str) -> None:
        super().__init__()
        D = cfg.head_dim
        self.head_dim, self.causal = D, causal
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, D, cfg.num_attention_heads, cfg.num_key_value_heads, bias=False,
                                          params_dtype=params_dtype, hf_legs=("to_q", "to_k", "to_v"),
                                          prefix=f"{prefix}.qkv_proj")
        if self.qkv_proj.num_kv_head_replicas != 1:
            raise ValueError("Cosmos3 tensor parallelism needs tp <= num_key_value_heads")
        self.to_out = RowParallelLinear(cfg.num_attention_heads * D, cfg.hidden_size, bias=False, params_dtype=params_dtype,
                                        prefix=f"{prefix}.to_out")
        self.norm_q = RMSNorm(D, cfg.rms_norm_eps, backend=norm_backend, dtype=params_dtype, prefix=f"{prefix}.norm_q")
        self.norm_k = RMSNorm(D, cfg.rms_norm_eps, backend=norm_backend, dtype=params_dtype, prefix=f"{prefix}.norm_k")
        self.num_local_heads, self.num_local_kv_heads = self.qkv_proj.num_heads, self.qkv_proj.num_kv_heads
        self.attn = Attention(self.num_local_heads, D, self.num_local_kv_heads, causal=causal, backend=attn_backend)
        self.eps = cfg.rms_norm_eps

    def project(self, x: torch.Tensor, cos_sin: torch.Tensor):
        """x (B, S, H), cos_sin (B, S, D) -> q (B,S,Hq,D), k, v (B,S,Hkv,D), normed and rotated."""
        B, S, _ = x.shape
        qkv, _ = self.qkv_proj(x)
        p = self.qkv_proj
        q, k, v = qkv.split([p.q_size, p.kv_size, p.kv_size], dim=-1)
        q = self.norm_q(q.reshape(B, S, -1, self.head_dim))
        k = self.norm_k(k.reshape(B, S, -1, self.head_dim))
        v = v.reshape(B, S, -1, self.head_dim)
        cs = cos_sin.reshape(B * S, -1)
        q = ref.apply_rope(q.reshape(B * S, -1, self.head_dim), cs).reshape(q.shape)
        k = ref.apply_rope(k.reshape(B * S, -1, self.head_dim), cs).reshape(k.shape)
        return q, k, v


class Cosmos3UndDecoderLayer(nn.Module):
    def __init__(self, cfg, *, attn_backend, norm_backend, params_dtype, prefix: str) -> None:
        super().__init__()
        nk = dict(backend=norm_backend, dtype=params_dtype)
        self.self_attn = Cosmos3Attention(cfg, causal=True, attn_backend=attn_backend, norm_backend=norm_backend,
                                          params_dtype=params_dtype, prefix=f"{prefix}.self_attn")
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, prefix=f"{prefix}.input_layernorm", **nk)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, prefix=f"{prefix}.post_attention_layernorm", **nk)
        self.mlp = DenseMLP(cfg.hidden_size, cfg.intermediate_size, gated=True, activation=cfg.hidden_act,
                            params_dtype=params_dtype, prefix=f"{prefix}.mlp")

    def forward(self, h: torch.Tensor, cos_sin: torch.Tensor):
        q, k, v = self.self_attn.project(self.input_layernorm(h), cos_sin)
        a = self.self_attn.attn(q, k, v)
        a, _ = self.self_attn.to_out(a.reshape(*h.shape[:-1], -1))
        h = h + a
        return h + self.mlp(self.post_attention_layernorm(h)), k, v


class Cosmos3GenDecoderLayer(nn.Module):
    def __init__(self, cfg, *, attn_backend, norm_backend, params_dtype, prefix: str) -> None:
        super().__init__()
        nk = dict(backend=norm_backend, dtype=params_dtype)
        self.cfg = cfg
        self.cross_attention = Cosmos3Attention(cfg, causal=False, attn_backend=attn_backend, norm_backend=norm_backend,
                                                params_dtype=params_dtype, prefix=f"{prefix}.cross_attention")
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, prefix=f"{prefix}.input_layernorm", **nk)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, prefix=f"{prefix}.post_attention_layernorm", **nk)
        self.mlp = DenseMLP(cfg.hidden_size, cfg.intermediate_size, gated=True, activation=cfg.hidden_act,
                            params_dtype=params_dtype, prefix=f"{prefix}.mlp")

    def forward(self, h: torch.Tensor, k_und: torch.Tensor, v_und: torch.Tensor, cos_sin: torch.Tensor) -> torch.Tensor:
        ca = self.cross_attention
        q, k, v = ca.project(self.input_layernorm(h), cos_sin)
        a = ca.attn(q, torch.cat([k_und, k], dim=1), torch.cat([v_und, v], dim=1))
        a, _ = ca.to_out(a.reshape(*h.shape[:-1], -1))
        h = h + a
        return h + self.mlp(self.post_attention_layernorm(h))

    # ---- B200 path: no concatenation, q/k norm + rope + KV placement in one kernel
    def forward_fused(self, h: torch.Tensor, kv_buf: tuple[torch.Tensor, torch.Tensor], s_text: int,
                      cos_sin: torch.Tensor, ws: "GenWorkspace") -> torch.Tensor:
        """h (B*S, H) bf16 on CUDA. ``kv_buf`` = (K, V) each (B*(s_text+S), Hkv, D) with the text K/V
        already in rows [b*(s_text+S), +s_text) of every sample; GEN K/V are written behind them."""
        ca, cfg = self.cross_attention, self.cfg
        B, S = ws.B, ws.S
        Hq, Hkv, D = ca.num_local_heads, ca.num_local_kv_heads, ca.head_dim
        kbuf, vbuf = kv_buf
        if ws.fp8 is not None:
            return self._forward_fused_fp8(h, kv_buf, cos_sin, ws)
        if ws.nvfp4 is not None:
            return self._forward_fused_nvfp4(h, kv_buf, cos_sin, ws)
        ops.norm(h, "rms", weight=self.input_layernorm.weight, eps=cfg.rms_norm_eps, out=ws.x)
        ops.gemm(ws.x, ca.qkv_proj.weight, ws.qkv)
        ops.rope_kv(ws.qkv, Hq, Hkv, D, ws.q, cos_sin=cos_sin, q_norm_w=ca.norm_q.weight, k_norm_w=ca.norm_k.weight,
                    norm_eps=cfg.rms_norm_eps, k_pool=kbuf, v_pool=vbuf, slots=ws.slots)
        ops.attention(ws.q.unflatten(1, (Hq, D)), kbuf, vbuf, ws.attn.unflatten(1, (Hq, D)), ws.q_start, ws.q_len,
                      ws.kv_ptr, ws.kv_len, max_q_len=S, sm_scale=D ** -0.5)
        if ca.to_out.tp_size > 1:
            part = ops.gemm(ws.attn, ca.to_out.weight, ws.part)
            h = h + P.all_reduce(part, axis=ca.to_out.axis)
        else:
            ops.gemm(ws.attn, ca.to_out.weight, h, residual=h)
        ops.norm(h, "rms", weight=self.post_attention_layernorm.weight, eps=cfg.rms_norm_eps, out=ws.x)
        ops.gemm(ws.x, self.mlp.gate_up_proj.weight, ws.act, act=self.mlp.activation, glu=True)
        if self.mlp.down_proj.tp_size > 1:
            part = ops.gemm(ws.act, self.mlp.down_proj.weight, ws.part)
            h = h + P.all_reduce(part, axis=self.mlp.down_proj.axis)
        else:
            ops.gemm(ws.act, self.mlp.down_proj.weight, h, residual=h)
        return h

    def _fp8_weights(self) -> dict:
        """Block-scaled e4m3 weights of this layer's four projections (stored ones of an fp8 checkpoint, else
        quantised once from the bf16 tensors)."""
        w = getattr(self, "_w8", None)
        if w is None:
            from ...ops.fp8_block import layer_weight_fp8

            ca = self.cross_attention
            w = {"qkv": layer_weight_fp8(ca.qkv_proj), "o": layer_weight_fp8(ca.to_out),
                 "gate_up": layer_weight_fp8(self.mlp.gate_up_proj), "down": layer_weight_fp8(self.mlp.down_proj)}
            self._w8 = w
        return w

    #: global scale of the activations on the NVFP4 path: block scales (ue4m3) are taken relative to it, which puts block
    #: maxima from 0.0015 to 336 inside their range
    NVFP4_ACT_GLOBAL = 0.125

    def _nvfp4_weights(self) -> dict:
        """e2m1 weights of the four projections with ue4m3 scales per 16 inputs in the interleaved layout and one fp32
        global scale each: taken from an NVFP4 checkpoint's layer as stored, else quantised once from bf16 by the same
        kernel that quantises activations."""
        w = getattr(self, "_w4", None)
        if w is None:
            from ...ops import nvfp4

            def prep(layer):
                if getattr(layer.spec, "spec_id", "") == "nvfp4_block_16":
                    K = layer.weight.shape[1] * 2
                    return layer.weight.data, nvfp4.swizzle_scales(layer.weight_scale.data, K), float(layer.weight_global_scale.item())
                wt = layer.weight.data.to(torch.bfloat16)
                g = max(float(wt.float().abs().amax().item()) / (6.0 * 448.0), 1e-12)
                q, sf = nvfp4.quantize_activation(wt.contiguous(), g, cached=False)
                return q, sf, g

            ca = self.cross_attention
            w = {"qkv": prep(ca.qkv_proj), "o": prep(ca.to_out), "gate_up": prep(self.mlp.gate_up_proj), "down": prep(self.mlp.down_proj)}
            self._w4 = w
        return w

    def _forward_fused_nvfp4(self, h: torch.Tensor, kv_buf, cos_sin: torch.Tensor, ws: "GenWorkspace") -> torch.Tensor:
        """The same layer with NVFP4 projections on the block-scaled tensor cores (reference: every linear of an NVFP4
        checkpoint through ``nvfp4_quantize`` + ``mm_fp4``, layers/linear/backends/flashinfer.py:163-200). Activations are
        quantised in front of each GEMM; the GEMM has no fused epilogue, so the residual add and the gated activation
        are passes of their own. Single GPU."""
        from ...ops import nvfp4

        ca, cfg, W = self.cross_attention, self.cfg, self._nvfp4_weights()
        S, ga = ws.S, self.NVFP4_ACT_GLOBAL
        Hq, Hkv, D = ca.num_local_heads, ca.num_local_kv_heads, ca.head_dim
        kbuf, vbuf = kv_buf

        def lin(x, name, out):
            q, sf = nvfp4.quantize_activation(x, ga)
            w4, sfw, gw = W[name]
            return nvfp4.gemm_nvfp4(q, sf, w4, sfw, ga * gw, out=out)

        ops.norm(h, "rms", weight=self.input_layernorm.weight, eps=cfg.rms_norm_eps, out=ws.x)
        lin(ws.x, "qkv", ws.qkv)
        ops.rope_kv(ws.qkv, Hq, Hkv, D, ws.q, cos_sin=cos_sin, q_norm_w=ca.norm_q.weight, k_norm_w=ca.norm_k.weight,
                    norm_eps=cfg.rms_norm_eps, k_pool=kbuf, v_pool=vbuf, slots=ws.slots)
        ops.attention(ws.q.unflatten(1, (Hq, D)), kbuf, vbuf, ws.attn.unflatten(1, (Hq, D)), ws.q_start, ws.q_len,
                      ws.kv_ptr, ws.kv_len, max_q_len=S, sm_scale=D ** -0.5)
        ops.axpy(h, lin(ws.attn, "o", ws.part), 1.0)
        ops.norm(h, "rms", weight=self.post_attention_layernorm.weight, eps=cfg.rms_norm_eps, out=ws.x)
        ops.gated_act(lin(ws.x, "gate_up", ws.nvfp4["gu"]), self.mlp.activation, interleaved=True, out=ws.act)
        ops.axpy(h, lin(ws.act, "down", ws.part), 1.0)
        return h

    def _forward_fused_fp8(self, h: torch.Tensor, kv_buf, cos_sin: torch.Tensor, ws: "GenWorkspace") -> torch.Tensor:
        """The same layer with block-scaled fp8 projections (reference: every linear through
        ``gemm_fp8_nt_groupwise`` with per-token activation quantisation, layers/linear/backends/flashinfer.py:132-157).
        The norm kernels emit the e4m3 rows and their 1 x 128 scales; attention output and the gated product pass
        through the quantiser; residual adds stay in the GEMM epilogues. Row-parallel sums over ``tp`` use NCCL."""
        from ...ops.fp8_block import gemm_fp8_block as g8, quantize_rows_into as q8

        ca, cfg, W, f = self.cross_attention, self.cfg, self._fp8_weights(), ws.fp8
        S = ws.S
        Hq, Hkv, D = ca.num_local_heads, ca.num_local_kv_heads, ca.head_dim
        kbuf, vbuf = kv_buf
        x8, xs, a8, as_, m8, ms = f["x"], f["xs"], f["attn"], f["attns"], f["act"], f["acts"]
        ops.norm(h, "rms", weight=self.input_layernorm.weight, eps=cfg.rms_norm_eps, out=ws.x, y8=x8, y8_scale=xs, y8_block=128)
        g8(x8, xs, *W["qkv"], ws.qkv)
        ops.rope_kv(ws.qkv, Hq, Hkv, D, ws.q, cos_sin=cos_sin, q_norm_w=ca.norm_q.weight, k_norm_w=ca.norm_k.weight,
                    norm_eps=cfg.rms_norm_eps, k_pool=kbuf, v_pool=vbuf, slots=ws.slots)
        ops.attention(ws.q.unflatten(1, (Hq, D)), kbuf, vbuf, ws.attn.unflatten(1, (Hq, D)), ws.q_start, ws.q_len,
                      ws.kv_ptr, ws.kv_len, max_q_len=S, sm_scale=D ** -0.5)
        q8(ws.attn, a8, as_)
        if ca.to_out.tp_size > 1:
            h = h + P.all_reduce(g8(a8, as_, *W["o"], ws.part), axis=ca.to_out.axis)
        else:
            g8(a8, as_, *W["o"], h, residual=h)
        ops.norm(h, "rms", weight=self.post_attention_layernorm.weight, eps=cfg.rms_norm_eps, out=ws.x, y8=x8, y8_scale=xs,
                 y8_block=128)
        g8(x8, xs, *W["gate_up"], ws.act, act=self.mlp.activation, glu=True)
        q8(ws.act, m8, ms)
        if self.mlp.down_proj.tp_size > 1:
            h = h + P.all_reduce(g8(m8, ms, *W["down"], ws.part), axis=self.mlp.down_proj.axis)
        else:
            g8(m8, ms, *W["down"], h, residual=h)
        return h

    def forward_fused_tp(self, h: torch.Tensor, y_in: torch.Tensor, wait, kv_buf, s_text: int, cos_sin: torch.Tensor,
                         ws: "GenWorkspace", next_norm_weight: torch.Tensor):
        """Tensor-parallel layer over peer memory. ``y_in`` is this layer's already normalised input (a
        gathered matrix other ranks may still be writing: ``wait`` makes the first GEMM wait for it);
        the residual ``h`` is kept only for the rows this rank owns. Each row-parallel product leaves
        its GEMM through the epilogue into the row owners' slots; the owner sums, adds the residual,
        applies the NEXT norm and stores the rows into every rank's gathered matrix, which the next
        GEMM waits on. Returns the ticket of the layer's output (normalised with ``next_norm_weight``)."""
        ca, cfg = self.cross_attention, self.cfg
        S = ws.S
        Hq, Hkv, D = ca.num_local_heads, ca.num_local_kv_heads, ca.head_dim
        kbuf, vbuf = kv_buf
        st = ws.stream
        scatter = h.shape[0] >= 1024
        ops.gemm(y_in, ca.qkv_proj.weight, ws.qkv, wait=wait)
        ops.rope_kv(ws.qkv, Hq, Hkv, D, ws.q, cos_sin=cos_sin, q_norm_w=ca.norm_q.weight, k_norm_w=ca.norm_k.weight,
                    norm_eps=cfg.rms_norm_eps, k_pool=kbuf, v_pool=vbuf, slots=ws.slots)
        ops.attention(ws.q.unflatten(1, (Hq, D)), kbuf, vbuf, ws.attn.unflatten(1, (Hq, D)), ws.q_start, ws.q_len,
                      ws.kv_ptr, ws.kv_len, max_q_len=S, sm_scale=D ** -0.5)
        t1 = st.linear_reduce(ws.attn, ca.to_out.weight, scatter=scatter, residual=h, norm="rms",
                              weight=self.post_attention_layernorm.weight, eps=cfg.rms_norm_eps, gather=True)
        ops.gemm(t1.y, self.mlp.gate_up_proj.weight, ws.act, act=self.mlp.activation, glu=True, wait=t1.wait)
        return st.linear_reduce(ws.act, self.mlp.down_proj.weight, scatter=scatter, residual=h, norm="rms",
                                weight=next_norm_weight, eps=cfg.rms_norm_eps, gather=True)


@dataclass
class GenWorkspace:
    """Static buffers of the fused GEN path for one (B, S, s_text) shape."""

    B: int
    S: int
    x: torch.Tensor
    qkv: torch.Tensor
    q: torch.Tensor
    attn: torch.Tensor
    act: torch.Tensor
    part: torch.Tensor
    slots: torch.Tensor
    q_start: torch.Tensor
    q_len: torch.Tensor
    kv_ptr: torch.Tensor
    kv_len: torch.Tensor
    stream: object | None = None   # PeerStream of the tensor-parallel group (None: single rank or NCCL fallback)
    fp8: dict | None = None        # block-scaled fp8 serving: e4m3 row buffers and 1 x 128 scales ("x", "attn", "act")
    nvfp4: dict | None = None      # NVFP4 serving: the un-gated gate/up product ("gu")


class Cosmos3LanguageModel(nn.Module):
    def __init__(self, cfg: Cosmos3Config, *, attn_backend, norm_backend, params_dtype, device, prefix: str = "language_model") -> None:
        super().__init__()
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, params_dtype=params_dtype, device=device,
                                                   prefix=f"{prefix}.embed_tokens")
        self.rotary_emb = MRotaryEmbedding(cfg.head_dim, cfg.mrope_section, cfg.rope_theta, interleaved=True)
        self.layers = nn.ModuleList([Cosmos3UndDecoderLayer(cfg, attn_backend=attn_backend, norm_backend=norm_backend,
                                                            params_dtype=params_dtype, prefix=f"{prefix}.layers.{i}")
                                     for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, backend=norm_backend, dtype=params_dtype, prefix=f"{prefix}.norm")
        self.norm.weight.optional = True        # loaded for parity, unused: only the K/V leave this tower

    def forward(self, text_ids: torch.Tensor, cos_sin: torch.Tensor):
        h = self.embed_tokens(text_ids)
        kv = []
        for layer in self.layers:
            h, k, v = layer(h, cos_sin)
            kv.append((k, v))
        return kv


@dataclass
class Cosmos3Condition:
    """Everything about a prompt that does not depend on the diffusion time."""

    cached_kv: list[tuple[torch.Tensor, torch.Tensor]]
    freqs_gen: torch.Tensor                      # (B, S_gen, head_dim) fp32 cos|sin
    video_shape: tuple[int, int, int]
    action_len: int = 0
    sound_len: int = 0
    fused: dict = field(default_factory=dict)    # lazily built buffers of the CUDA path

    def refresh_from(self, new: "Cosmos3Condition") -> None:
        """Take over another prompt of the same geometry in place: the rotary table and the text K/V rows of the
        CUDA path's buffers are overwritten where they are, so that a captured step which reads them serves the
        new prompt. A different text length or latent geometry is refused (it needs buffers of its own)."""
        same = (new.video_shape == self.video_shape and new.action_len == self.action_len and new.sound_len == self.sound_len
                and new.freqs_gen.shape == self.freqs_gen.shape and len(new.cached_kv) == len(self.cached_kv)
                and new.cached_kv[0][0].shape == self.cached_kv[0][0].shape)
        if not same:
            raise ValueError("refresh_from needs a condition of the same text length and latent geometry")
        self.freqs_gen.copy_(new.freqs_gen)
        for (k_old, v_old), (k_new, v_new) in zip(self.cached_kv, new.cached_kv):
            k_old.copy_(k_new)
            v_old.copy_(v_new)
        for _, bufs in self.fused.values():
            for (kb, vb), (k_new, v_new) in zip(bufs, new.cached_kv):
                B, s_text, Hkv, D = k_new.shape
                kb.view(B, -1, Hkv, D)[:, :s_text].copy_(k_new)
                vb.view(B, -1, Hkv, D)[:, :s_text].copy_(v_new)


__all__ = ["compute_mrope_position_ids_text", "compute_mrope_position_ids_vision", "local_head_counts",
           "TimestepEmbedder", "DomainAwareLinear", "Cosmos3Attention", "Cosmos3UndDecoderLayer",
           "Cosmos3GenDecoderLayer", "Cosmos3LanguageModel", "Cosmos3Condition", "GenWorkspace"]
