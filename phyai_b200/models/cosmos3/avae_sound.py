"""Sound decoder of Cosmos3: latent frames (25 Hz, 64 channels) -> stereo waveform (48 kHz).

A stack of transposed-convolution upsamplers (total hop = product of the strides), each followed
by three dilated residual units with Snake activations. Checkpoint convolutions are weight-normed;
the ``(g, v)`` pairs are folded into plain weights while loading, so inference runs ordinary convs.

Reference: phyai/src/phyai/models/cosmos3/avae_sound.py:15-190.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from ...layers.activation import Snake1d
from ...layers.conv import Conv1d, ConvTranspose1d
from .configuration_cosmos3 import Cosmos3AVAESoundConfig


def _sub(prefix: str, name: str) -> str:
    return f"{prefix}.{name}" if prefix else ""


class DilatedUnit(nn.Module):
    """x + conv1x1(snake(conv7_dilated(snake(x))))."""

    def __init__(self, dim: int, dilation: int, *, prefix: str = "", **kw) -> None:
        super().__init__()
        self.snake1 = Snake1d(dim, prefix=_sub(prefix, "snake1"), **kw)
        self.conv1 = Conv1d(dim, dim, 7, dilation=dilation, padding=3 * dilation, weight_norm=True,
                            prefix=_sub(prefix, "conv1"), **kw)
        self.snake2 = Snake1d(dim, prefix=_sub(prefix, "snake2"), **kw)
        self.conv2 = Conv1d(dim, dim, 1, weight_norm=True, prefix=_sub(prefix, "conv2"), **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.conv2(self.snake2(self.conv1(self.snake1(x))))
        trim = (x.shape[-1] - y.shape[-1]) // 2
        return (x[..., trim:-trim] if trim > 0 else x) + y


class UpsampleStage(nn.Module):
    def __init__(self, cin: int, cout: int, stride: int, *, prefix: str = "", **kw) -> None:
        super().__init__()
        self.snake1 = Snake1d(cin, prefix=_sub(prefix, "snake1"), **kw)
        self.conv_t1 = ConvTranspose1d(cin, cout, 2 * stride, stride=stride, padding=math.ceil(stride / 2),
                                       output_padding=stride % 2, weight_norm=True, prefix=_sub(prefix, "conv_t1"), **kw)
        for i, d in enumerate((1, 3, 9), start=1):
            setattr(self, f"res_unit{i}", DilatedUnit(cout, d, prefix=_sub(prefix, f"res_unit{i}"), **kw))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.conv_t1(self.snake1(x))
        return self.res_unit3(self.res_unit2(self.res_unit1(x)))


class WaveDecoder(nn.Module):
    def __init__(self, width: int, latent_ch: int, audio_ch: int, strides, mults, *, prefix: str = "", **kw) -> None:
        super().__init__()
        mults = [1, *mults]
        n = len(strides)
        self.conv1 = Conv1d(latent_ch, width * mults[-1], 7, padding=3, weight_norm=True, prefix=_sub(prefix, "conv1"), **kw)
        self.block = nn.ModuleList([UpsampleStage(width * mults[n - i], width * mults[n - i - 1], s,
                                                  prefix=_sub(prefix, f"block.{i}"), **kw) for i, s in enumerate(strides)])
        self.snake1 = Snake1d(width, prefix=_sub(prefix, "snake1"), **kw)
        self.conv2 = Conv1d(width, audio_ch, 7, padding=3, bias=False, weight_norm=True, prefix=_sub(prefix, "conv2"), **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.conv1(x)
        for stage in self.block:
            x = stage(x)
        return self.conv2(self.snake1(x))


class Cosmos3AVAESoundDecoder(nn.Module):
    def __init__(self, config: Cosmos3AVAESoundConfig, *, dtype: torch.dtype | None = None, device=None) -> None:
        if not isinstance(config, Cosmos3AVAESoundConfig):
            raise TypeError(f"expected Cosmos3AVAESoundConfig, got {type(config).__name__}")
        super().__init__()
        kw = {k: v for k, v in (("dtype", dtype), ("device", device)) if v is not None}
        self.config = config
        self.latent_ch, self.audio_channels, self.sample_rate = config.latent_ch, config.audio_channels, config.sample_rate
        self.hop_size = math.prod(config.dec_strides)
        self.decoder = WaveDecoder(config.dec_dim, config.latent_ch, config.audio_channels,
                                   list(reversed(config.dec_strides)), list(config.dec_c_mults), prefix="decoder", **kw)

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        """(B, latent_ch, T) -> (B, audio_channels, T * hop_size) in [-1, 1]."""
        return self.decoder(latent).clamp(-1.0, 1.0)


def cosmos3_avae_weight_remap(key: str) -> str | None:
    """Only the decode path is built: keep ``decoder.*`` (names match the checkpoint), drop the encoder."""
    return key if key.startswith("decoder.") else None


__all__ = ["Cosmos3AVAESoundDecoder", "WaveDecoder", "cosmos3_avae_weight_remap"]
