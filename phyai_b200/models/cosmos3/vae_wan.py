"""WAN 2.2 video VAE (16x spatial, 4x temporal, 48 latent channels) for Cosmos3.

The network is causal in time. It is written as a *stream*: every temporal convolution
keeps the last ``k_t - 1`` input frames in a :class:`StreamState`, so a clip can be pushed
through in one piece (the default: 180 GB of HBM holds a 720p clip's activations, and one
pass keeps the convolutions large) or in temporal chunks of any size with bit-identical
maths. The first frame of a stream is special in the two places the architecture makes it
so: temporal upsampling leaves it un-doubled, and temporal downsampling passes it through.

Parameter names equal the ``AutoencoderKLWan`` checkpoint keys, so loading needs only a
filter. ``decode_parallel`` splits the latent grid into spatial tiles with a halo, one per
rank of the ``cfg x tp`` group, decodes them concurrently and cross-fades the overlaps.

Reference: phyai/src/phyai/models/cosmos3/vae_wan.py:55-1074.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...layers.conv import Conv2d, Conv3d
from .configuration_cosmos3 import Cosmos3WanVAEConfig


class StreamState:
    """Temporal context carried between chunks of one clip."""

    def __init__(self) -> None:
        self.tails: dict[int, torch.Tensor] = {}
        self.first = True  # the chunk being processed starts with the clip's first frame


def _param(shape, prefix: str, init: float, device, dtype) -> nn.Parameter:
    p = nn.Parameter(torch.full(shape, init, device=device, dtype=dtype), requires_grad=False)
    if prefix:
        p.hf_keys = {prefix: None}
    return p


class CausalConv3d(Conv3d):
    """3-D convolution padded symmetrically in space and only on the past side in time."""

    def __init__(self, cin: int, cout: int, kernel, *, stride=1, padding=0, causal: bool = True, prefix: str = "", **kw):
        super().__init__(cin, cout, kernel, stride=stride, padding=0, prefix=prefix, **kw)
        pt, ph, pw = (padding,) * 3 if isinstance(padding, int) else padding
        self._space_pad = (pw, pw, ph, ph)
        self._past = 2 * pt if causal else 0  # frames of history the kernel wants

    def forward(self, x: torch.Tensor, state: StreamState | None = None) -> torch.Tensor:  # type: ignore[override]
        if self._past:
            tail = state.tails.get(id(self)) if state is not None else None
            if tail is None:
                tail = x.new_zeros(x.shape[0], x.shape[1], self._past, *x.shape[3:])
            x = torch.cat([tail, x], dim=2)
            if state is not None:
                state.tails[id(self)] = x[:, :, -self._past:].clone()
        if any(self._space_pad):
            x = F.pad(x, self._space_pad)
        return super().forward(x)


class ChannelNorm(nn.Module):
    """L2-normalise over channels, scale by sqrt(C) and a learned gain (no epsilon in the mean)."""

    def __init__(self, dim: int, *, images: bool, prefix: str = "", device=None, dtype=None) -> None:
        super().__init__()
        shape = (dim, 1, 1) if images else (dim, 1, 1, 1)
        self.scale = float(dim) ** 0.5
        self.gamma = _param(shape, f"{prefix}.gamma" if prefix else "", 1.0, device, dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.normalize(x, dim=1) * self.scale * self.gamma.to(x.dtype)


def _per_frame(fn, x: torch.Tensor) -> torch.Tensor:
    b, c, t, h, w = x.shape
    y = fn(x.transpose(1, 2).reshape(b * t, c, h, w))
    return y.reshape(b, t, *y.shape[1:]).transpose(1, 2)


class Resample(nn.Module):
    """Spatial x2 up/down sampling, optionally with the temporal x2 step of the causal stream."""

    def __init__(self, dim: int, mode: str, *, out_dim: int | None = None, prefix: str = "", **kw) -> None:
        super().__init__()
        if mode not in ("upsample2d", "upsample3d", "downsample2d", "downsample3d"):
            raise ValueError(f"unknown resample mode {mode!r}")
        self.mode, self.up, self.temporal = mode, mode.startswith("up"), mode.endswith("3d")
        conv_prefix = f"{prefix}.resample.1" if prefix else ""
        if self.up:
            self.conv = Conv2d(dim, dim // 2 if out_dim is None else out_dim, 3, padding=1, prefix=conv_prefix, **kw)
            if self.temporal:
                self.time_conv = CausalConv3d(dim, 2 * dim, (3, 1, 1), padding=(1, 0, 0),
                                              prefix=f"{prefix}.time_conv" if prefix else "", **kw)
        else:
            self.conv = Conv2d(dim, dim, 3, stride=2, pad_sides=(0, 1, 0, 1), prefix=conv_prefix, **kw)
            if self.temporal:
                self.time_conv = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), causal=False,
                                              prefix=f"{prefix}.time_conv" if prefix else "", **kw)

    def _time_up(self, x: torch.Tensor, state: StreamState | None) -> torch.Tensor:
        first = state is None or state.first
        head, rest = (x[:, :, :1], x[:, :, 1:]) if first else (None, x)
        parts = [] if head is None else [head]
        if rest.shape[2]:
            b, c, t, h, w = rest.shape
            y = self.time_conv(rest, state).reshape(b, 2, c, t, h, w)
            parts.append(torch.stack((y[:, 0], y[:, 1]), dim=3).reshape(b, c, 2 * t, h, w))
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=2)

    def _time_down(self, x: torch.Tensor, state: StreamState | None) -> torch.Tensor:
        first = state is None or state.first
        key = id(self)
        if first:
            seq, head = x, x[:, :, :1]
        else:
            seq, head = torch.cat([state.tails[key], x], dim=2), None
        if state is not None:
            state.tails[key] = x[:, :, -1:].clone()
        if seq.shape[2] < 3:
            return head
        if (seq.shape[2] - 1) % 2:
            raise ValueError("temporal downsampling takes 1 + 2k frames per stream position")
        y = self.time_conv(seq)
        return y if head is None else torch.cat([head, y], dim=2)

    def forward(self, x: torch.Tensor, state: StreamState | None = None) -> torch.Tensor:
        if self.up:
            if self.temporal:
                x = self._time_up(x, state)
            up = lambda f: self.conv(F.interpolate(f.float(), scale_factor=2.0, mode="nearest-exact").to(f.dtype))  # noqa: E731
            return _per_frame(up, x)
        x = _per_frame(self.conv, x)
        return self._time_down(x, state) if self.temporal else x


class ResidualBlock(nn.Module):
    def __init__(self, cin: int, cout: int, *, prefix: str = "", **kw) -> None:
        super().__init__()
        p = (lambda s: f"{prefix}.{s}") if prefix else (lambda s: "")
        nkw = {k: kw[k] for k in ("device", "dtype") if k in kw}
        self.norm1 = ChannelNorm(cin, images=False, prefix=p("norm1"), **nkw)
        self.conv1 = CausalConv3d(cin, cout, 3, padding=1, prefix=p("conv1"), **kw)
        self.norm2 = ChannelNorm(cout, images=False, prefix=p("norm2"), **nkw)
        self.conv2 = CausalConv3d(cout, cout, 3, padding=1, prefix=p("conv2"), **kw)
        self.conv_shortcut = CausalConv3d(cin, cout, 1, prefix=p("conv_shortcut"), **kw) if cin != cout else None

    def forward(self, x: torch.Tensor, state: StreamState | None = None) -> torch.Tensor:
        skip = x if self.conv_shortcut is None else self.conv_shortcut(x)
        x = self.conv1(F.silu(self.norm1(x)), state)
        x = self.conv2(F.silu(self.norm2(x)), state)
        return x + skip


class FrameAttention(nn.Module):
    """Single-head self-attention over the H*W positions of each frame (head width = channels)."""

    def __init__(self, dim: int, *, prefix: str = "", **kw) -> None:
        super().__init__()
        p = (lambda s: f"{prefix}.{s}") if prefix else (lambda s: "")
        nkw = {k: kw[k] for k in ("device", "dtype") if k in kw}
        self.norm = ChannelNorm(dim, images=True, prefix=p("norm"), **nkw)
        self.to_qkv = Conv2d(dim, 3 * dim, 1, prefix=p("to_qkv"), **kw)
        self.proj = Conv2d(dim, dim, 1, prefix=p("proj"), **kw)

    def _frames(self, f: torch.Tensor) -> torch.Tensor:
        n, c, h, w = f.shape
        q, k, v = self.to_qkv(self.norm(f)).reshape(n, 3, c, h * w).transpose(2, 3).unsqueeze(2).unbind(1)
        o = F.scaled_dot_product_attention(q, k, v)  # (n, 1, hw, c)
        return self.proj(o.squeeze(1).transpose(1, 2).reshape(n, c, h, w))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + _per_frame(self._frames, x)


class MidBlock(nn.Module):
    def __init__(self, dim: int, *, prefix: str = "", **kw) -> None:
        super().__init__()
        p = (lambda s: f"{prefix}.{s}") if prefix else (lambda s: "")
        self.resnets = nn.ModuleList([ResidualBlock(dim, dim, prefix=p("resnets.0"), **kw),
                                      ResidualBlock(dim, dim, prefix=p("resnets.1"), **kw)])
        self.attentions = nn.ModuleList([FrameAttention(dim, prefix=p("attentions.0"), **kw)])

    def forward(self, x: torch.Tensor, state: StreamState | None = None) -> torch.Tensor:
        x = self.resnets[0](x, state)
        return self.resnets[1](self.attentions[0](x), state)


def spread_up(x: torch.Tensor, cout: int, ft: int, fs: int, drop_first: bool) -> torch.Tensor:
    """Parameter-free up shortcut: repeat channels, then unfold the repeats into (t, h, w) factors."""
    b, c, t, h, w = x.shape
    rep = cout * ft * fs * fs // c
    y = x.repeat_interleave(rep, dim=1).reshape(b, cout, ft, fs, fs, t, h, w)
    y = y.permute(0, 1, 5, 2, 6, 3, 7, 4).reshape(b, cout, t * ft, h * fs, w * fs)
    return y[:, :, ft - 1:] if drop_first else y


def pool_down(x: torch.Tensor, cout: int, ft: int, fs: int) -> torch.Tensor:
    """Parameter-free down shortcut: fold (t, h, w) factors into channels, average channel groups."""
    front = (-x.shape[2]) % ft
    if front:
        x = F.pad(x, (0, 0, 0, 0, front, 0))
    b, c, t, h, w = x.shape
    y = x.reshape(b, c, t // ft, ft, h // fs, fs, w // fs, fs).permute(0, 1, 3, 5, 7, 2, 4, 6)
    y = y.reshape(b, cout, c * ft * fs * fs // cout, t // ft, h // fs, w // fs)
    return y.mean(dim=2)


class UpBlock(nn.Module):
    def __init__(self, cin: int, cout: int, n_res: int, *, up: bool, temporal: bool, prefix: str = "", **kw) -> None:
        super().__init__()
        p = (lambda s: f"{prefix}.{s}") if prefix else (lambda s: "")
        self.cout, self.ft = cout, 2 if temporal else 1
        self.resnets = nn.ModuleList([ResidualBlock(cin if j == 0 else cout, cout, prefix=p(f"resnets.{j}"), **kw)
                                      for j in range(n_res + 1)])
        self.upsampler = (Resample(cout, "upsample3d" if temporal else "upsample2d", out_dim=cout,
                                   prefix=p("upsampler"), **kw) if up else None)

    def forward(self, x: torch.Tensor, state: StreamState | None = None) -> torch.Tensor:
        skip = x
        for r in self.resnets:
            x = r(x, state)
        if self.upsampler is None:
            return x
        x = self.upsampler(x, state)
        return x + spread_up(skip, self.cout, self.ft, 2, drop_first=state is None or state.first)


class DownBlock(nn.Module):
    def __init__(self, cin: int, cout: int, n_res: int, *, down: bool, temporal: bool, prefix: str = "", **kw) -> None:
        super().__init__()
        p = (lambda s: f"{prefix}.{s}") if prefix else (lambda s: "")
        self.cout, self.ft, self.fs = cout, 2 if temporal else 1, 2 if down else 1
        self.resnets = nn.ModuleList([ResidualBlock(cin if j == 0 else cout, cout, prefix=p(f"resnets.{j}"), **kw)
                                      for j in range(n_res)])
        self.downsampler = (Resample(cout, "downsample3d" if temporal else "downsample2d", prefix=p("downsampler"), **kw)
                            if down else None)

    def forward(self, x: torch.Tensor, state: StreamState | None = None) -> torch.Tensor:
        skip = x
        for r in self.resnets:
            x = r(x, state)
        if self.downsampler is not None:
            x = self.downsampler(x, state)
        return x + pool_down(skip, self.cout, self.ft, self.fs)


class Encoder3d(nn.Module):
    def __init__(self, cin: int, dim: int, z_out: int, dim_mult, n_res: int, temporal_down, *, prefix: str = "", **kw):
        super().__init__()
        p = (lambda s: f"{prefix}.{s}") if prefix else (lambda s: "")
        nkw = {k: kw[k] for k in ("device", "dtype") if k in kw}
        dims = [dim] + [dim * m for m in dim_mult]
        self.conv_in = CausalConv3d(cin, dims[0], 3, padding=1, prefix=p("conv_in"), **kw)
        last = len(dim_mult) - 1
        self.down_blocks = nn.ModuleList([
            DownBlock(a, b, n_res, down=i != last, temporal=i != last and bool(temporal_down[i]),
                      prefix=p(f"down_blocks.{i}"), **kw) for i, (a, b) in enumerate(zip(dims[:-1], dims[1:]))])
        self.mid_block = MidBlock(dims[-1], prefix=p("mid_block"), **kw)
        self.norm_out = ChannelNorm(dims[-1], images=False, prefix=p("norm_out"), **nkw)
        self.conv_out = CausalConv3d(dims[-1], z_out, 3, padding=1, prefix=p("conv_out"), **kw)

    def forward(self, x: torch.Tensor, state: StreamState | None = None) -> torch.Tensor:
        x = self.conv_in(x, state)
        for blk in self.down_blocks:
            x = blk(x, state)
        x = self.mid_block(x, state)
        return self.conv_out(F.silu(self.norm_out(x)), state)


class Decoder3d(nn.Module):
    def __init__(self, dim: int, z_dim: int, dim_mult, n_res: int, temporal_up, cout: int, *, prefix: str = "", **kw):
        super().__init__()
        p = (lambda s: f"{prefix}.{s}") if prefix else (lambda s: "")
        nkw = {k: kw[k] for k in ("device", "dtype") if k in kw}
        dims = [dim * dim_mult[-1]] + [dim * m for m in reversed(dim_mult)]
        self.conv_in = CausalConv3d(z_dim, dims[0], 3, padding=1, prefix=p("conv_in"), **kw)
        self.mid_block = MidBlock(dims[0], prefix=p("mid_block"), **kw)
        last = len(dim_mult) - 1
        self.up_blocks = nn.ModuleList([
            UpBlock(a, b, n_res, up=i != last, temporal=i != last and bool(temporal_up[i]),
                    prefix=p(f"up_blocks.{i}"), **kw) for i, (a, b) in enumerate(zip(dims[:-1], dims[1:]))])
        self.norm_out = ChannelNorm(dims[-1], images=False, prefix=p("norm_out"), **nkw)
        self.conv_out = CausalConv3d(dims[-1], cout, 3, padding=1, prefix=p("conv_out"), **kw)

    def forward(self, x: torch.Tensor, state: StreamState | None = None) -> torch.Tensor:
        x = self.mid_block(self.conv_in(x, state), state)
        for blk in self.up_blocks:
            x = blk(x, state)
        return self.conv_out(F.silu(self.norm_out(x)), state)


def fold_patches(x: torch.Tensor, p: int) -> torch.Tensor:
    """(B, C, T, H, W) -> (B, C*p*p, T, H/p, W/p); channel order (c, w-offset, h-offset)."""
    if p == 1:
        return x
    b, c, t, h, w = x.shape
    if h % p or w % p:
        raise ValueError(f"H={h} and W={w} must be multiples of the patch size {p}")
    return x.reshape(b, c, t, h // p, p, w // p, p).permute(0, 1, 6, 4, 2, 3, 5).reshape(b, c * p * p, t, h // p, w // p)


def unfold_patches(x: torch.Tensor, p: int) -> torch.Tensor:
    if p == 1:
        return x
    b, cp, t, h, w = x.shape
    c = cp // (p * p)
    return x.reshape(b, c, p, p, t, h, w).permute(0, 1, 4, 5, 3, 6, 2).reshape(b, c, t, h * p, w * p)


def tile_grid(n: int) -> tuple[int, int]:
    """Most nearly square (rows, cols) with rows * cols == n and rows <= cols."""
    rows = max(r for r in range(1, math.isqrt(n) + 1) if n % r == 0)
    return rows, n // rows


def tile_span(length: int, n: int, idx: int, halo: int) -> tuple[int, int]:
    """Slice of ``length`` decoded by tile ``idx`` of ``n``: its own share widened by ``halo`` inside the image."""
    return max(0, idx * length // n - halo), min(length, (idx + 1) * length // n + halo)


def feather_1d(n: int, width: int, device, dtype) -> torch.Tensor:
    """Blend weight that ramps over ``width`` samples at both ends and is 1 between them."""
    if width <= 0 or n <= 1:
        return torch.ones(n, device=device, dtype=dtype)
    i = torch.arange(n, device=device, dtype=torch.float32)
    return torch.minimum((i + 1) / (width + 1), (n - i) / (width + 1)).clamp(max=1.0).to(dtype)


class Cosmos3WanVAE(nn.Module):
    def __init__(self, config: Cosmos3WanVAEConfig, *, device=None, dtype=None) -> None:
        if not isinstance(config, Cosmos3WanVAEConfig):
            raise TypeError(f"expected Cosmos3WanVAEConfig, got {type(config).__name__}")
        super().__init__()
        kw = {k: v for k, v in (("device", device), ("dtype", dtype)) if v is not None}
        self.config = config
        z = config.z_dim
        self.z_dim, self.patch_size = z, config.patch_size
        self.scale_factor_temporal, self.scale_factor_spatial = config.scale_factor_temporal, config.scale_factor_spatial
        self.encoder = Encoder3d(config.out_channels, config.base_dim, 2 * z, config.dim_mult, config.num_res_blocks,
                                 config.temperal_downsample, prefix="encoder", **kw)
        self.quant_conv = CausalConv3d(2 * z, 2 * z, 1, prefix="quant_conv", **kw)
        self.post_quant_conv = CausalConv3d(z, z, 1, prefix="post_quant_conv", **kw)
        self.decoder = Decoder3d(config.decoder_base_dim, z, config.dim_mult, config.num_res_blocks,
                                 tuple(reversed(config.temperal_downsample)), config.out_channels, prefix="decoder", **kw)
        mean = torch.tensor(list(config.latents_mean) if config.latents_mean is not None else [0.0] * z)
        std = torch.tensor(list(config.latents_std) if config.latents_std is not None else [1.0] * z)
        self.register_buffer("latents_mean", mean.view(1, z, 1, 1, 1), persistent=False)
        self.register_buffer("latents_std", std.view(1, z, 1, 1, 1), persistent=False)

    # ---- decode
    @torch.no_grad()
    def decode(self, latents: torch.Tensor, *, frames_per_chunk: int | None = None) -> torch.Tensor:
        """(B, z, t, h, w) normalised latents -> (B, 3, 1 + 4(t-1), 16h, 16w) pixels in [-1, 1].

        ``frames_per_chunk`` bounds the activation memory by streaming that many latent frames at a
        time; ``None`` runs the clip in one pass. Both give the same result.
        """
        x = self.post_quant_conv(latents * self.latents_std.to(latents) + self.latents_mean.to(latents))
        t = x.shape[2]
        if frames_per_chunk is None or frames_per_chunk >= t:
            out = self.decoder(x, None)
        else:
            state, parts, i = StreamState(), [], 0
            while i < t:
                parts.append(self.decoder(x[:, :, i:i + frames_per_chunk], state))
                state.first = False
                i += frames_per_chunk
            out = torch.cat(parts, dim=2)
        return unfold_patches(out, self.patch_size).clamp(-1.0, 1.0)

    @torch.no_grad()
    def decode_parallel(self, latents: torch.Tensor, *, halo: int = 2, frames_per_chunk: int | None = None) -> torch.Tensor:
        """Spatially tiled decode over the ranks of ``cfg x tp``; every rank returns the full clip."""
        from ... import parallel as P

        mesh = P.default_mesh()
        axes = [(ax, mesh.axis_size(ax), mesh.axis_local_rank(ax)) for ax in ("cfg", "tp")
                if mesh is not None and mesh.has_axis(ax)]
        n = math.prod(s for _, s, _ in axes) if axes else 1
        if n <= 1:
            return self.decode(latents, frames_per_chunk=frames_per_chunk)
        me = 0
        for _, size, r in axes:  # cfg outer, tp inner
            me = me * size + r
        rows, cols = tile_grid(n)
        h_lat, w_lat = latents.shape[-2:]
        s = self.scale_factor_spatial
        spans = [(tile_span(h_lat, rows, k // cols, halo), tile_span(w_lat, cols, k % cols, halo)) for k in range(n)]
        (h0, h1), (w0, w1) = spans[me]
        mine = self.decode(latents[..., h0:h1, w0:w1].contiguous(), frames_per_chunk=frames_per_chunk)
        # tile extents are a pure function of (shape, n): no metadata exchange, one padded gather per axis
        th, tw = max(a[1] - a[0] for a, _ in spans) * s, max(b[1] - b[0] for _, b in spans) * s
        buf = mine.new_zeros(*mine.shape[:3], th, tw)
        buf[..., :mine.shape[-2], :mine.shape[-1]] = mine
        tiles = buf[None]
        for ax, size, _ in reversed(axes):
            if size > 1:
                tiles = P.all_gather(tiles[None].contiguous(), axis=ax, dim=0, mesh=mesh).reshape(-1, *buf.shape)
        acc = mine.new_zeros(*mine.shape[:3], h_lat * s, w_lat * s, dtype=torch.float32)
        wsum = torch.zeros(h_lat * s, w_lat * s, device=mine.device, dtype=torch.float32)
        for k, ((a0, a1), (b0, b1)) in enumerate(spans):
            hh, ww = (a1 - a0) * s, (b1 - b0) * s
            wgt = feather_1d(hh, halo * s, mine.device, torch.float32)[:, None] * feather_1d(ww, halo * s, mine.device, torch.float32)
            acc[..., a0 * s:a1 * s, b0 * s:b1 * s] += tiles[k, ..., :hh, :ww].float() * wgt
            wsum[a0 * s:a1 * s, b0 * s:b1 * s] += wgt
        return (acc / wsum.clamp_min(1e-6)).clamp(-1.0, 1.0).to(mine.dtype)

    decode_tp = decode_parallel

    # ---- encode
    @torch.no_grad()
    def encode(self, pixels: torch.Tensor, *, sample: bool = False, generator: torch.Generator | None = None,
               frames_per_chunk: int | None = None) -> torch.Tensor:
        """(B, 3, 1 + 4k, H, W) in [-1, 1] -> normalised latents (B, z, 1 + k, H/16, W/16) (posterior mean unless ``sample``)."""
        x = fold_patches(pixels, self.patch_size)
        t = x.shape[2]
        if (t - 1) % self.scale_factor_temporal:
            raise ValueError(f"encode takes 1 + {self.scale_factor_temporal}k frames, got {t}")
        if frames_per_chunk is None or frames_per_chunk >= t:
            h = self.encoder(x, None)
        else:
            step = max(self.scale_factor_temporal, frames_per_chunk // self.scale_factor_temporal * self.scale_factor_temporal)
            # the first frame alone seeds the stream; the rest follows in multiples of the temporal factor
            state, i = StreamState(), 1
            parts = [self.encoder(x[:, :, :1], state)]
            state.first = False
            while i < t:
                parts.append(self.encoder(x[:, :, i:i + step], state))
                i += step
            h = torch.cat(parts, dim=2)
        mean, logvar = self.quant_conv(h).chunk(2, dim=1)
        if sample:
            std = torch.exp(0.5 * logvar.clamp(-30.0, 20.0))
            mean = mean + std * torch.randn(mean.shape, generator=generator, device=mean.device, dtype=mean.dtype)
        return (mean - self.latents_mean.to(mean)) / self.latents_std.to(mean)


def decode_auto(vae: Cosmos3WanVAE, latents: torch.Tensor) -> torch.Tensor:
    """Tile-parallel decode when a multi-rank ``cfg``/``tp`` mesh is active, plain decode otherwise."""
    return vae.decode_parallel(latents)


_VAE_ROOTS = ("encoder.", "decoder.", "quant_conv.", "post_quant_conv.")


def cosmos3_vae_weight_remap(key: str) -> str | None:
    """Parameter names already equal the ``AutoencoderKLWan`` keys: keep the four sub-trees, drop the rest."""
    return key if key.startswith(_VAE_ROOTS) else None


__all__ = ["Cosmos3WanVAE", "Encoder3d", "Decoder3d", "StreamState", "CausalConv3d", "cosmos3_vae_weight_remap",
           "decode_auto", "fold_patches", "unfold_patches", "tile_grid", "tile_span", "feather_1d"]
