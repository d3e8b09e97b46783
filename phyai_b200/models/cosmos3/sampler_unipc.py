"""UniPC multistep sampler (order 2, ``bh2``, data prediction) on flow-matching sigmas.

Every coefficient of a UniPC step depends only on the sigma schedule, never on the data,
so ``set_timesteps`` reduces the schedule to a table of scalar weights (computed in float64
on the host) and ``step`` is a handful of fused multiply-adds over the latent:

    x0_t   = x - sigma_t * v                        (model output -> data prediction)
    x_corr = c_x * x_last + c_0 * x0_{t-1} + c_1 * x0_{t-2} + c_t * x0_t     (corrector, from step 1)
    x_next = p_x * x      + p_0 * x0_t     + p_1 * x0_{t-1}                  (predictor)

Schedules: Karras sigmas (0.147 .. 200, rho 7) mapped by ``s / (s + 1)``, or linear flow
sigmas warped by ``flow_shift``. Behavioural parity with
phyai/src/phyai/models/cosmos3/sampler_unipc.py:16-288 (which evaluates the same formulas with
tensor scalars inside every step, including a 2x2 ``linalg.solve``).
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch


def resolve_use_karras_sigmas(value: bool | None, ckpt: str | Path | None = None) -> bool:
    """Explicit value, else ``scheduler/scheduler_config.json``'s flag, else True."""
    if value is not None:
        return bool(value)
    if ckpt is None:
        return True
    f = Path(ckpt) / "scheduler" / "scheduler_config.json"
    if f.is_file():
        try:
            return bool(json.loads(f.read_text()).get("use_karras_sigmas", True))
        except (ValueError, OSError):
            return True
    return True


def _lam(sigma: float) -> float:
    a = 1.0 - sigma
    if sigma <= 0.0:
        return math.inf
    if a <= 0.0:
        return -math.inf
    return math.log(a) - math.log(sigma)


@dataclass(frozen=True)
class StepCoeffs:
    sigma: float
    # corrector (None on the first step): x = c_x*x_last + c_0*m_prev + c_1*m_prev2 + c_t*m_this
    corr: tuple[float, float, float, float] | None
    # predictor: x_next = p_x*x + p_0*m_this + p_1*m_prev
    pred: tuple[float, float, float]


class UniPCMultistepSampler:
    def __init__(self, *, num_train_timesteps: int = 1000, solver_order: int = 2, sigma_min: float = 0.147,
                 sigma_max: float = 200.0, karras_rho: float = 7.0, flow_shift: float = 1.0,
                 use_karras_sigmas: bool = True, lower_order_final: bool = True) -> None:
        if solver_order not in (1, 2):
            raise ValueError("UniPC here supports solver_order 1 or 2")
        self.num_train_timesteps, self.solver_order = int(num_train_timesteps), int(solver_order)
        self.sigma_min, self.sigma_max, self.karras_rho = float(sigma_min), float(sigma_max), float(karras_rho)
        self.flow_shift, self.use_karras_sigmas = float(flow_shift), bool(use_karras_sigmas)
        self.lower_order_final = bool(lower_order_final)
        self.sigmas: torch.Tensor | None = None
        self.timesteps: torch.Tensor | None = None
        self.table: list[StepCoeffs] = []
        self.num_inference_steps: int | None = None
        self._reset_state()

    def _reset_state(self) -> None:
        self._step_index: int | None = None
        self._m: list[torch.Tensor | None] = [None, None]    # x0 predictions: [t-2, t-1]
        self._last_sample: torch.Tensor | None = None

    @property
    def step_index(self) -> int | None:
        return self._step_index

    # -------------------------------------------------------------- schedule
    def set_timesteps(self, num_inference_steps: int, device: torch.device | str | None = None) -> None:
        n = int(num_inference_steps)
        if self.use_karras_sigmas:
            ramp = np.linspace(0, 1, n)
            lo, hi = self.sigma_min ** (1 / self.karras_rho), self.sigma_max ** (1 / self.karras_rho)
            s = (hi + ramp * (lo - hi)) ** self.karras_rho
            s = s / (s + 1.0)
        else:
            sh = self.flow_shift
            base = 1.0 - np.linspace(1.0, 1.0 / self.num_train_timesteps, self.num_train_timesteps)[::-1]
            base = sh * base / (1.0 + (sh - 1.0) * base)
            s = np.linspace(float(base[0]), float(base[-1]), n + 1)[:-1]
            s = sh * s / (1.0 + (sh - 1.0) * s)
        self.timesteps = torch.from_numpy((s * self.num_train_timesteps).copy()).to(device=device, dtype=torch.int64)
        sig = np.concatenate([s, [0.0]]).astype(np.float32)       # stored in fp32, as checkpoints' schedulers do
        self.sigmas = torch.from_numpy(sig)
        self.num_inference_steps = n
        self.table = self._build_table([float(v) for v in sig], n)
        self._reset_state()

    def _build_table(self, sig: list[float], n: int) -> list[StepCoeffs]:
        table: list[StepCoeffs] = []
        lower = 0            # how many earlier outputs exist (capped at solver_order)
        prev_order = 0
        for i in range(n):
            corr = None
            if i > 0:
                corr = self._corrector(sig, i, prev_order)
            order = min(self.solver_order, n - i) if self.lower_order_final else self.solver_order
            order = min(order, lower + 1)
            pred = self._predictor(sig, i, order)
            table.append(StepCoeffs(sig[i], corr, pred))
            prev_order = order
            lower = min(lower + 1, self.solver_order)
        return table

    @staticmethod
    def _predictor(sig: list[float], i: int, order: int) -> tuple[float, float, float]:
        s_t, s_0 = sig[i + 1], sig[i]
        a_t = 1.0 - s_t
        h = _lam(s_t) - _lam(s_0)
        e = math.expm1(-h)                       # h_phi_1 and B(h) for bh2
        p_x, p_0, p_1 = s_t / s_0, -a_t * e, 0.0
        if order == 2:
            rk = (_lam(sig[i - 1]) - _lam(s_0)) / h
            w = -a_t * e * 0.5 / rk              # applied to (m_prev - m_this)
            p_0, p_1 = p_0 - w, w
        return p_x, p_0, p_1

    @staticmethod
    def _corrector(sig: list[float], i: int, order: int) -> tuple[float, float, float, float]:
        s_t, s_0 = sig[i], sig[i - 1]
        a_t = 1.0 - s_t
        h = _lam(s_t) - _lam(s_0)
        hh = -h
        e = math.expm1(hh)
        phi_k = e / hh - 1.0
        c_x, base0 = s_t / s_0, -a_t * e
        if order <= 1:
            r_last, r_prev, rk = 0.5, 0.0, 1.0
        else:
            rk = (_lam(sig[i - 2]) - _lam(s_0)) / h
            b1 = phi_k / e
            b2 = (phi_k / hh - 0.5) * 2.0 / e
            # solve [[1, 1], [rk, 1]] @ [r_prev, r_last] = [b1, b2]
            det = 1.0 - rk
            r_prev = (b1 - b2) / det
            r_last = (b2 - rk * b1) / det
        # x = c_x*x_last + base0*m0 - a_t*e*( r_prev*(m1 - m0)/rk + r_last*(m_t - m0) )
        k = -a_t * e
        c_1 = k * r_prev / rk if order > 1 else 0.0
        c_t = k * r_last
        c_0 = base0 - c_1 - c_t
        return c_x, c_0, c_1, c_t

    # ------------------------------------------------------------------ step
    def convert_model_output(self, model_output: torch.Tensor, sample: torch.Tensor) -> torch.Tensor:
        return sample - self.table[self._step_index].sigma * model_output

    def step(self, model_output: torch.Tensor, timestep: torch.Tensor | int | None, sample: torch.Tensor) -> torch.Tensor:
        if self.num_inference_steps is None:
            raise RuntimeError("call set_timesteps() before step()")
        if self._step_index is None:
            self._step_index = 0
        c = self.table[self._step_index]
        m_t = sample - c.sigma * model_output
        m_prev, m_prev2 = self._m[1], self._m[0]
        if c.corr is not None and self._last_sample is not None:
            c_x, c_0, c_1, c_t = c.corr
            x = c_x * self._last_sample + c_0 * m_prev + c_t * m_t
            if c_1 != 0.0 and m_prev2 is not None:
                x = x + c_1 * m_prev2
            sample = x.to(sample.dtype)
        self._m = [m_prev, m_t]
        self._last_sample = sample
        p_x, p_0, p_1 = c.pred
        out = p_x * sample + p_0 * m_t
        if p_1 != 0.0 and m_prev is not None:
            out = out + p_1 * m_prev
        self._step_index += 1
        return out.to(sample.dtype)


class FusedUniPCStream:
    """One latent stream of a denoise loop updated on the device by ``ops.unipc_step``: a single kernel per step
    in place of the dozen tensor ops of :meth:`UniPCMultistepSampler.step` (and of the guidance combine and the
    clean-frame copy around it). State (last corrected sample, two x0 predictions) is fp32; the sample stays bf16.

    ``sample`` is read as ``[B, C, T, inner]`` (``view`` = (C, T, inner)); ``keep`` ``[B, T]`` marks frames that are
    put back from ``cond`` after every update; innermost columns from ``live_inner`` on get a zero velocity.
    The coefficient table is the sampler's (reference update: phyai/src/phyai/models/cosmos3/sampler_unipc.py:145-288)."""

    def __init__(self, sampler: UniPCMultistepSampler, sample: torch.Tensor, *, view: tuple[int, int, int] | None = None,
                 keep: torch.Tensor | None = None, cond: torch.Tensor | None = None, live_inner: int = 0) -> None:
        if not (sample.is_cuda and sample.dtype == torch.bfloat16 and sample.is_contiguous()):
            raise ValueError("the fused sampler updates a contiguous bf16 CUDA sample in place")
        if sampler.num_inference_steps is None:
            raise RuntimeError("call set_timesteps() on the sampler first")
        self.table, self.sample, self.i = sampler.table, sample, 0
        self.view = view if view is not None else (1, 1, sample.shape[-1])
        self.live_inner = int(live_inner)
        z = lambda: torch.zeros(sample.shape, dtype=torch.float32, device=sample.device)  # noqa: E731
        self.x_last, self.m1, self.m2 = z(), z(), z()
        self.keep = self.cond = None
        if keep is not None:
            if cond is None:
                raise ValueError("keep needs the clean values")
            self.keep = keep.to(device=sample.device, dtype=torch.uint8).contiguous()
            self.cond = cond.to(device=sample.device, dtype=torch.bfloat16).expand_as(sample).contiguous()

    @staticmethod
    def usable(sample: torch.Tensor) -> bool:
        return sample.is_cuda and sample.dtype == torch.bfloat16

    def step(self, velocity: torch.Tensor, *, uncond: torch.Tensor | None = None, g: float = 1.0) -> torch.Tensor:
        """``velocity`` already guided, or the conditional one with ``uncond`` and ``g`` for an in-kernel combine."""
        from ... import ops

        if self.i >= len(self.table):
            raise RuntimeError("more sampler steps than timesteps")
        c = self.table[self.i]
        v = velocity.to(torch.bfloat16).contiguous()
        u = None if uncond is None else uncond.to(torch.bfloat16).contiguous()
        ops.unipc_step(v, self.sample, self.x_last, self.m1, self.m2, sigma=c.sigma, corr=c.corr, pred=c.pred, v_uncond=u, g=g,
                       keep=self.keep, cond=self.cond, view=self.view, live_inner=self.live_inner)
        self.i += 1
        return self.sample


__all__ = ["UniPCMultistepSampler", "StepCoeffs", "FusedUniPCStream", "resolve_use_karras_sigmas"]
