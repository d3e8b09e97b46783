"""``Cosmos3Transformer``: patchify, condition encoding, the per-step GEN pass, checkpoint remap.

Reference: phyai/src/phyai/models/cosmos3/modeling_cosmos3.py:615-1135.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ... import parallel as P
from ...engine_config import get_engine_config, resolve_engine_defaults
from ...env import envs
from ...layers.layer_norm import RMSNorm
from ...layers.linear import ReplicatedLinear
from .configuration_cosmos3 import Cosmos3Config
from .modeling_cosmos3 import (Cosmos3Condition, Cosmos3GenDecoderLayer, Cosmos3LanguageModel, DomainAwareLinear,
                               GenWorkspace, TimestepEmbedder, compute_mrope_position_ids_text,
                               compute_mrope_position_ids_vision)


class Cosmos3Transformer(nn.Module):
    def __init__(self, config: Cosmos3Config, *, params_dtype=None, attn_backend=None, norm_backend=None, device=None) -> None:
        super().__init__()
        dtype, attn_backend, norm_backend = resolve_engine_defaults(params_dtype, attn_backend, norm_backend)
        device = device if device is not None else get_engine_config().device.target
        self.config, self.params_dtype = config, dtype
        kw = dict(attn_backend=attn_backend, norm_backend=norm_backend, params_dtype=dtype)
        self.language_model = Cosmos3LanguageModel(config, device=device, **kw)
        self.gen_layers = nn.ModuleList([Cosmos3GenDecoderLayer(config, prefix=f"gen_layers.{i}", **kw)
                                         for i in range(config.num_hidden_layers)])
        self.norm_moe_gen = RMSNorm(config.hidden_size, config.rms_norm_eps, backend=norm_backend, dtype=dtype, prefix="norm_moe_gen")
        self.proj_in = ReplicatedLinear(config.patch_latent_dim, config.hidden_size, bias=True, params_dtype=dtype, prefix="proj_in")
        self.proj_out = ReplicatedLinear(config.hidden_size, config.patch_latent_dim, bias=True, params_dtype=dtype, prefix="proj_out")
        self.time_embedder = TimestepEmbedder(config.hidden_size, params_dtype=dtype, device=device, prefix="time_embedder")
        if config.action_gen:
            self.action_proj_in = DomainAwareLinear(config.action_dim, config.hidden_size, config.num_embodiment_domains,
                                                    params_dtype=dtype, device=device, prefix="action_proj_in")
            self.action_proj_out = DomainAwareLinear(config.hidden_size, config.action_dim, config.num_embodiment_domains,
                                                     params_dtype=dtype, device=device, prefix="action_proj_out")
            self.action_modality_embed = nn.Parameter(torch.zeros(config.hidden_size, dtype=dtype, device=device), requires_grad=False)
            self.action_modality_embed.hf_keys = {"action_modality_embed": None}
        if config.sound_gen:
            self.audio_proj_in = ReplicatedLinear(config.sound_dim, config.hidden_size, bias=True, params_dtype=dtype, prefix="audio_proj_in")
            self.audio_proj_out = ReplicatedLinear(config.hidden_size, config.sound_dim, bias=True, params_dtype=dtype, prefix="audio_proj_out")
            self.audio_modality_embed = nn.Parameter(torch.zeros(config.hidden_size, dtype=dtype, device=device), requires_grad=False)
            self.audio_modality_embed.hf_keys = {"audio_modality_embed": None}
        self.use_fused = (torch.device(device).type == "cuda" and dtype == torch.bfloat16
                          and get_engine_config().resolved_backend("attn") == "b200")
        self.use_peer = envs.PHYAI_PEER_COMM.get()   # tensor-parallel GEN layers over peer memory (else NCCL all-reduce)
        # generation tower in block-scaled fp8 (e4m3 weights with 128 x 128 scales, activations per 1 x 128 block);
        # the peer-memory tensor-parallel layer is bf16 only, so fp8 + tp sums its row-parallel products over NCCL
        self.serve_fp8 = bool(envs.PHYAI_COSMOS3_FP8.get())
        # generation tower in NVFP4 (e2m1 with ue4m3 scales per 16 inputs) on the block-scaled tensor cores; one GPU only
        self.serve_nvfp4 = bool(envs.PHYAI_COSMOS3_NVFP4.get())

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> "Cosmos3Transformer":
        on_gpu = next(self.parameters()).is_cuda   # billions of values: draw them where they live
        g = torch.Generator(device=next(self.parameters()).device if on_gpu else "cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() == 1 and ("norm" in name) and "bias" not in name:
                continue
            if on_gpu:
                p.copy_(torch.randn(p.shape, generator=g, device=p.device, dtype=torch.float32).mul_(std).to(p.dtype))
            else:
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
        return self

    # ---------------------------------------------------------------- patches
    def _pad_to_patch_size(self, h: int, w: int) -> tuple[int, int, int, int]:
        p = self.config.latent_patch_size
        hp, wp = (h + p - 1) // p, (w + p - 1) // p
        return hp, wp, hp * p, wp * p

    def patchify(self, latents: torch.Tensor, t: int, h: int, w: int) -> torch.Tensor:
        """(B, C, t, h, w) -> (B, t*hp*wp, p*p*C), patch vector ordered (py, px, c)."""
        B, p, c = latents.shape[0], self.config.latent_patch_size, self.config.latent_channel
        hp, wp, h_pad, w_pad = self._pad_to_patch_size(h, w)
        if (h_pad, w_pad) != (h, w):
            latents = F.pad(latents, (0, w_pad - w, 0, h_pad - h))
        x = latents.reshape(B, c, t, hp, p, wp, p).permute(0, 2, 3, 5, 4, 6, 1)
        return x.reshape(B, t * hp * wp, p * p * c)

    def unpatchify(self, tokens: torch.Tensor, t: int, h: int, w: int) -> torch.Tensor:
        B, p, c = tokens.shape[0], self.config.latent_patch_size, self.config.latent_channel
        hp, wp, h_pad, w_pad = self._pad_to_patch_size(h, w)
        x = tokens.reshape(B, t, hp, wp, p, p, c).permute(0, 6, 1, 2, 4, 3, 5).reshape(B, c, t, h_pad, w_pad)
        return x[:, :, :, :h, :w] if (h_pad, w_pad) != (h, w) else x

    # -------------------------------------------------------------- condition
    def _rope_tables(self, text_mask: torch.Tensor, t: int, hp: int, wp: int, fps, device, *, action_len=0, sound_len=0,
                     sound_fps=None) -> tuple[torch.Tensor, torch.Tensor]:
        """fp32 ``cos | sin`` tables (B, S_text, D) and (B, S_gen, D)."""
        cfg = self.config
        B, s_text = text_mask.shape
        lens = text_mask.sum(dim=1).long().tolist()
        eff_fps = fps if fps is not None and t > 1 else None
        eff_sfps = sound_fps if sound_fps is not None and sound_len > 1 else None
        text_pos, gen_pos = [], []
        for b in range(B):
            tp, off = compute_mrope_position_ids_text(int(lens[b]), 0)
            media = off + cfg.temporal_modality_margin
            vp, _ = compute_mrope_position_ids_vision(t, hp, wp, media, fps=eff_fps, base_fps=cfg.base_fps,
                                                      temporal_compression_factor=cfg.temporal_compression_factor,
                                                      enable_fps_modulation=cfg.enable_fps_modulation)
            if lens[b] < s_text:
                tp = torch.cat([tp, torch.zeros(3, s_text - lens[b], dtype=tp.dtype)], dim=1)
            text_pos.append(tp.float())
            vp = vp.float()
            if action_len > 0:
                ap, _ = compute_mrope_position_ids_vision(action_len, 1, 1, media, fps=eff_fps, base_fps=cfg.base_fps,
                                                          temporal_compression_factor=1,
                                                          base_temporal_compression_factor=cfg.temporal_compression_factor,
                                                          enable_fps_modulation=cfg.enable_fps_modulation, start_frame_offset=1)
                vp = torch.cat([vp, ap.float()], dim=1)
            if sound_len > 0:
                sp, _ = compute_mrope_position_ids_vision(sound_len, 1, 1, media, fps=eff_sfps, base_fps=cfg.base_fps,
                                                          temporal_compression_factor=1,
                                                          enable_fps_modulation=cfg.enable_fps_modulation, start_frame_offset=0)
                vp = torch.cat([vp, sp.float()], dim=1)
            gen_pos.append(vp)
        rope = self.language_model.rotary_emb
        und = torch.stack([rope.cos_sin(p.to(device)) for p in text_pos])
        gen = torch.stack([rope.cos_sin(p.to(device)) for p in gen_pos])
        return und, gen

    @torch.no_grad()
    def encode_condition(self, text_ids: torch.Tensor, text_mask: torch.Tensor, video_shape: tuple[int, int, int],
                         fps: float | None = None, *, action_len: int = 0, sound_len: int = 0,
                         sound_fps: float | None = None) -> Cosmos3Condition:
        """Run the UND tower once over the prompt and build the GEN rope table."""
        t, h, w = video_shape
        hp, wp, _, _ = self._pad_to_patch_size(h, w)
        lens = text_mask.sum(dim=1)
        real = int(lens.max().item())
        if int(lens.min().item()) != real:
            raise ValueError("Cosmos3 requires identical real text lengths within a batch")
        und, gen = self._rope_tables(text_mask, t, hp, wp, fps, text_ids.device, action_len=action_len,
                                     sound_len=sound_len, sound_fps=sound_fps)
        kv = self.language_model(text_ids, und)
        kv = [(k[:, :real].contiguous(), v[:, :real].contiguous()) for k, v in kv]
        return Cosmos3Condition(kv, gen.contiguous(), video_shape, action_len, sound_len)

    # ----------------------------------------------------------------- forward
    @staticmethod
    def _gate_timestep(time_embed: torch.Tensor, mask: torch.Tensor | None, per_frame: int) -> torch.Tensor:
        if mask is None:
            return time_embed[:, None]
        gate = mask.to(time_embed.dtype).repeat_interleave(per_frame, dim=1)[..., None]
        return time_embed[:, None] * gate

    def _fused_state(self, cond: Cosmos3Condition, B: int, S: int, device) -> tuple[GenWorkspace, list]:
        """Buffers of the CUDA path, built once per condition: K/V buffers with the text K/V in place."""
        key = (B, S)
        if key in cond.fused:
            return cond.fused[key]
        cfg = self.config
        ca = self.gen_layers[0].cross_attention
        Hq, Hkv, D = ca.num_local_heads, ca.num_local_kv_heads, ca.head_dim
        s_text = cond.cached_kv[0][0].shape[1]
        tot = s_text + S
        bf = torch.bfloat16
        z = lambda *s: torch.empty(*s, dtype=bf, device=device)  # noqa: E731
        ar = torch.arange(B, dtype=torch.int32, device=device)
        slots = (torch.arange(B, device=device)[:, None] * tot + s_text + torch.arange(S, device=device)[None]).reshape(-1)
        ws = GenWorkspace(B, S, z(B * S, cfg.hidden_size), z(B * S, (Hq + 2 * Hkv) * D), z(B * S, Hq * D), z(B * S, Hq * D),
                          z(B * S, self.gen_layers[0].mlp.down_proj.input_size_per_partition), z(B * S, cfg.hidden_size),
                          slots.long(), ar * S, torch.full_like(ar, S), ar * tot, torch.full_like(ar, tot))
        tp = self.gen_layers[0].mlp.down_proj.tp_size
        if self.serve_fp8:
            f8, f32 = torch.float8_e4m3fn, torch.float32
            widths = {"x": cfg.hidden_size, "attn": Hq * D, "act": self.gen_layers[0].mlp.down_proj.input_size_per_partition}
            if any(w % 128 for w in widths.values()):
                raise ValueError(f"block-scaled fp8 needs per-rank widths that are multiples of 128, got {widths}")
            ws.fp8 = {}
            for name, w in widths.items():
                ws.fp8[name] = torch.empty(B * S, w, dtype=f8, device=device)
                ws.fp8[name + "s"] = torch.empty(B * S, w // 128, dtype=f32, device=device)
        if self.serve_nvfp4 and not self.serve_fp8:
            from ...ops import nvfp4

            if tp > 1 or not nvfp4.available():
                raise RuntimeError("NVFP4 serving needs the phyai_b200._blockscaled module and a single tensor-parallel rank")
            if cfg.hidden_size % 32 or (Hq * D) % 32 or self.gen_layers[0].mlp.down_proj.input_size_per_partition % 32:
                raise ValueError("NVFP4 needs projection inputs that are multiples of 32")
            ws.nvfp4 = {"gu": torch.empty(B * S, 2 * self.gen_layers[0].mlp.down_proj.input_size_per_partition, dtype=bf, device=device)}
        if tp > 1 and self.use_peer and not self.serve_fp8:
            from ...parallel.symm import PeerGroup

            rows, H = B * S, cfg.hidden_size
            per = -(-rows // tp) if rows >= 1024 else rows
            need = 2 * tp * per * H * 2 + rows * H * 2 + (64 << 20)
            pg = PeerGroup.for_axis(P.default_mesh(), self.gen_layers[0].mlp.down_proj.axis, heap_bytes=max(need, 1 << 30))
            ws.stream = pg.stream(f"cosmos3.gen:{rows}", per, H, gather_rows=rows, gather_cols=H)
        bufs = []
        for k_und, v_und in cond.cached_kv:
            kb = torch.zeros(B * tot, Hkv, D, dtype=bf, device=device)
            vb = torch.zeros_like(kb)
            kb.view(B, tot, Hkv, D)[:, :s_text].copy_(k_und)
            vb.view(B, tot, Hkv, D)[:, :s_text].copy_(v_und)
            bufs.append((kb, vb))
        cond.fused[key] = (ws, bufs)
        return ws, bufs

    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor, timestep: torch.Tensor, condition: Cosmos3Condition, *,
                noisy_frame_mask: torch.Tensor | None = None, action_latents: torch.Tensor | None = None,
                action_domain_id: torch.Tensor | None = None, action_noisy_mask: torch.Tensor | None = None,
                sound_latents: torch.Tensor | None = None, sound_noisy_mask: torch.Tensor | None = None):
        """Velocity of the video latents ``(B, C, t, h, w)`` [and of the action / sound stream]."""
        cfg = self.config
        t, h, w = condition.video_shape
        hp, wp, _, _ = self._pad_to_patch_size(h, w)
        hv, _ = self.proj_in(self.patchify(hidden_states, t, h, w))
        te = self.time_embedder(timestep * cfg.timestep_scale).to(hv.dtype)
        hg = hv + self._gate_timestep(te, noisy_frame_mask, hp * wp)
        s_video = hg.shape[1]
        if action_latents is not None:
            if action_latents.shape[1] != condition.action_len:
                raise ValueError(f"action_latents length {action_latents.shape[1]} != condition.action_len {condition.action_len}")
            a = self.action_proj_in(action_latents, action_domain_id) + self.action_modality_embed.to(hv.dtype)
            hg = torch.cat([hg, a + self._gate_timestep(te, action_noisy_mask, 1)], dim=1)
        if sound_latents is not None:
            if action_latents is not None:
                raise NotImplementedError("Cosmos3 does not co-generate action and sound in one forward")
            if sound_latents.shape[1] != condition.sound_len:
                raise ValueError(f"sound_latents length {sound_latents.shape[1]} != condition.sound_len {condition.sound_len}")
            s, _ = self.audio_proj_in(sound_latents)
            s = s + self.audio_modality_embed.to(hv.dtype)
            hg = torch.cat([hg, s + self._gate_timestep(te, sound_noisy_mask, 1)], dim=1)
        B, S, H = hg.shape
        normed = False
        if self.use_fused and hg.is_cuda:
            ws, bufs = self._fused_state(condition, B, S, hg.device)
            s_text = condition.cached_kv[0][0].shape[1]
            cs = condition.freqs_gen.reshape(B * S, -1)
            x = hg.reshape(B * S, H).contiguous()
            if ws.stream is not None:
                # sequence-parallel residual: every layer hands the next one its already normalised input
                y, wait = ops.norm(x, "rms", weight=self.gen_layers[0].input_layernorm.weight, eps=cfg.rms_norm_eps, out=ws.x), None
                n = len(self.gen_layers)
                for i, (layer, kv) in enumerate(zip(self.gen_layers, bufs)):
                    nxt = self.gen_layers[i + 1].input_layernorm.weight if i + 1 < n else self.norm_moe_gen.weight
                    tk = layer.forward_fused_tp(x, y, wait, kv, s_text, cs, ws, nxt)
                    y, wait = tk.y, tk.wait
                hg = ws.stream.wait_gather(tk).reshape(B, S, H)
                normed = True
            else:
                for layer, kv in zip(self.gen_layers, bufs):
                    x = layer.forward_fused(x, kv, s_text, cs, ws)
                hg = x.reshape(B, S, H)
        else:
            for layer, (k_und, v_und) in zip(self.gen_layers, condition.cached_kv):
                hg = layer(hg, k_und, v_und, condition.freqs_gen)
        if not normed:
            hg = self.norm_moe_gen(hg)
        vo, _ = self.proj_out(hg[:, :s_video])
        video_vel = self.unpatchify(vo, t, h, w)
        if action_latents is not None:
            return video_vel, self.action_proj_out(hg[:, s_video:], action_domain_id)
        if sound_latents is not None:
            so, _ = self.audio_proj_out(hg[:, s_video:])
            return video_vel, so
        return video_vel


# ----------------------------------------------------------- checkpoint remap
_UND_LEAF = {k: k for k in ("self_attn.to_q", "self_attn.to_k", "self_attn.to_v", "self_attn.to_out", "self_attn.norm_q",
                            "self_attn.norm_k", "input_layernorm", "post_attention_layernorm", "mlp.gate_proj",
                            "mlp.up_proj", "mlp.down_proj")}
_GEN_LEAF = {
    "self_attn.add_q_proj": "cross_attention.to_q", "self_attn.add_k_proj": "cross_attention.to_k",
    "self_attn.add_v_proj": "cross_attention.to_v", "self_attn.to_add_out": "cross_attention.to_out",
    "self_attn.norm_added_q": "cross_attention.norm_q", "self_attn.norm_added_k": "cross_attention.norm_k",
    "input_layernorm_moe_gen": "input_layernorm", "post_attention_layernorm_moe_gen": "post_attention_layernorm",
    "mlp_moe_gen.gate_proj": "mlp.gate_proj", "mlp_moe_gen.up_proj": "mlp.up_proj", "mlp_moe_gen.down_proj": "mlp.down_proj",
}
_TOP = ("proj_in.", "proj_out.", "time_embedder.", "norm_moe_gen.", "action_proj_in.", "action_proj_out.",
        "action_modality_embed", "audio_proj_in.", "audio_proj_out.", "audio_modality_embed")


def cosmos3_weight_remap(key: str) -> str | None:
    """``transformer/`` checkpoint key -> parameter key (``None`` drops it). A shared ``layers.{i}.<leaf>``
    source goes to the UND tower (``language_model.layers.{i}``) or the GEN tower (``gen_layers.{i}``) by leaf."""
    if key.startswith("lm_head."):
        return None
    if key.startswith("embed_tokens.") or key.startswith("norm."):
        return f"language_model.{key}"
    if key.startswith(_TOP):
        return key
    if key.startswith("layers."):
        idx, leaf = key[len("layers."):].split(".", 1)
        tail = ""
        for suf in (".weight", ".bias"):
            if leaf.endswith(suf):
                leaf, tail = leaf[: -len(suf)], suf
                break
        if leaf in _UND_LEAF:
            return f"language_model.layers.{idx}.{_UND_LEAF[leaf]}{tail}"
        if leaf in _GEN_LEAF:
            return f"gen_layers.{idx}.{_GEN_LEAF[leaf]}{tail}"
    return None


def cosmos3_inverse_remap(param_key: str) -> str:
    """Parameter key -> upstream checkpoint key (used by the synthetic checkpoint writer)."""
    if param_key.startswith("language_model.layers."):
        return param_key[len("language_model."):]
    if param_key.startswith("language_model."):
        return param_key[len("language_model."):]
    if param_key.startswith("gen_layers."):
        idx, leaf = param_key[len("gen_layers."):].split(".", 1)
        tail = ""
        for suf in (".weight", ".bias"):
            if leaf.endswith(suf):
                leaf, tail = leaf[: -len(suf)], suf
                break
        inv = {v: k for k, v in _GEN_LEAF.items()}
        return f"layers.{idx}.{inv[leaf]}{tail}"
    return param_key


__all__ = ["Cosmos3Transformer", "cosmos3_weight_remap", "cosmos3_inverse_remap"]
