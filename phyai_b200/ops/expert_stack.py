"""Host side of the persistent action-expert kernel (``csrc/expert_stack.cu``).

:class:`ExpertStack` owns what one launch needs besides the model weights: the tensor maps of
the four projection weights of every block, the per-(step, layer) fp32 vectors that replace the
norm kernels (column factors ``1 + scale``, branch gates, ``shift @ W^T`` biases), and the
L2-resident scratch the phases exchange results through. :meth:`run` issues ONE cooperative
launch that advances the Euler loop from ``step_begin`` to ``step_end``; it allocates nothing
and is safe inside a stream capture.

The kernel covers one robot (up to 64 action rows), head dim 256, one KV head and a KV range of
at most ``64 * splits`` rows; :func:`ExpertStack.supports` tells whether a geometry fits. The loop it
replaces in the reference: phyai/src/phyai/models/pi05/model_runner_pi05.py:689-738.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ext


@dataclass
class ExpertGeometry:
    rows: int            # action rows M
    hidden: int
    inter: int
    q_heads: int
    head_dim: int
    action_dim: int
    layers: int
    steps: int


class ExpertStack:
    ROWS = 64

    def __init__(self, geo: ExpertGeometry, *, device: torch.device | str = "cuda") -> None:
        self.geo, self.device = geo, torch.device(device)
        grid = int(ext().expert_stack_grid())
        if grid <= 0:
            raise RuntimeError("expert_stack: the kernel cannot be made resident on this device")
        self.grid = grid
        self.splits = min(18, grid // geo.q_heads)
        g = geo
        nqkv = (g.q_heads + 2) * g.head_dim
        n = self.ROWS * (g.action_dim + g.hidden + nqkv + 2 * g.inter + 2) + g.q_heads * self.splits * self.ROWS * (g.head_dim + 2)
        self.scratch = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.attn = torch.zeros(self.ROWS, g.q_heads * g.head_dim, dtype=torch.bfloat16, device=self.device)
        self.barrier = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.tmaps: torch.Tensor | None = None
        self._keep: list[torch.Tensor] = []
        self.tables: dict[str, torch.Tensor] = {}
        self.debug = 0      # timing experiments only (bit 0: plain stores instead of reductions: wrong results)

    # ------------------------------------------------------------------ capability
    @staticmethod
    def supports(geo: ExpertGeometry, max_kv_rows: int) -> bool:
        """True when one launch can serve this geometry on the current device."""
        try:
            grid = int(ext().expert_stack_grid())
        except Exception:
            return False
        if grid < 128 or geo.rows > ExpertStack.ROWS or geo.head_dim != 256:
            return False
        if geo.hidden % 128 or geo.inter % 64 or geo.action_dim % 4:
            return False
        splits = min(18, grid // geo.q_heads)
        # a unit holds ceil(pool rows / splits) + ceil(rows / splits) <= 64 keys, at most 8 of them new
        pool_rows = max(0, max_kv_rows - geo.rows)
        if splits <= 0 or -(-geo.rows // splits) > 8 or -(-pool_rows // splits) + -(-geo.rows // splits) > 64:
            return False
        nt = [(geo.q_heads + 2) * geo.head_dim // 128, geo.hidden // 128, 2 * geo.inter // 128, geo.hidden // 128]
        kb = [geo.hidden // 64, geo.q_heads * geo.head_dim // 64, geo.hidden // 64, geo.inter // 64]
        for a, b in zip(nt, kb):
            total = a * b
            for c in range(grid):
                p0, p1 = total * c // grid, total * (c + 1) // grid
                if p1 - p0 > 8 or (p1 > p0 and (p1 - 1) // b - p0 // b + 1 > 3):
                    return False
        return True

    # ------------------------------------------------------------------ set-up
    def set_weights(self, layer_weights: list[tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]]) -> None:
        """``(qkv, o, gate_up, down)`` bf16 weights per block, in checkpoint row order (gate / up interleaved)."""
        flat = [w for ws in layer_weights for w in ws]
        self._keep = flat
        self.tmaps = ext().expert_stack_tmaps(flat, self.attn)

    def set_tables(self, *, in_scale, post_scale, gate_in, gate_post, qkv_bias, gu_bias, fin_scale, out_bias) -> None:
        """fp32 vectors indexed ``[step][layer][...]`` (``fin_scale`` / ``out_bias``: ``[step][...]``)."""
        t = dict(in_scale=in_scale, post_scale=post_scale, gate_in=gate_in, gate_post=gate_post, qkv_bias=qkv_bias,
                 gu_bias=gu_bias, fin_scale=fin_scale, out_bias=out_bias)
        self.tables = {k: v.to(self.device, torch.float32).contiguous() for k, v in t.items()}

    # ------------------------------------------------------------------ launch
    def run(self, *, w_in, b_in, w_out, k_pool, v_pool, kv_ptr, kv_len, pos, cos_sin, x0, out, eps: float, dt: float,
            sm_scale: float, step_begin: int = 0, step_end: int | None = None, trace: torch.Tensor | None = None) -> None:
        g = self.geo
        if self.tmaps is None or not self.tables:
            raise RuntimeError("expert_stack: set_weights / set_tables first")
        ext().expert_stack_run(self.tmaps, g.rows, g.hidden, g.inter, g.q_heads, g.head_dim, g.action_dim, g.layers,
                               step_begin, g.steps if step_end is None else step_end, self.splits, eps, dt, sm_scale,
                               self.tables["in_scale"], self.tables["post_scale"], self.tables["gate_in"],
                               self.tables["gate_post"], self.tables["qkv_bias"], self.tables["gu_bias"],
                               self.tables["fin_scale"], self.tables["out_bias"], w_in, b_in, w_out, k_pool, v_pool,
                               kv_ptr, kv_len, pos, cos_sin, x0, out, self.scratch, self.attn, self.barrier, trace, self.debug)


__all__ = ["ExpertStack", "ExpertGeometry"]
