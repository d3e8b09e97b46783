"""Python face of the sm_100a kernels in ``phyai_b200/csrc``.

Every function here launches exactly one hand-written CUDA kernel on the current
stream and allocates nothing unless the caller leaves ``out=None``. The module
refuses to work without the compiled extension: there is no eager fallback on a
GPU, so a missing build fails loudly instead of silently running PyTorch ops.
``phyai_b200.ops.ref`` holds plain PyTorch fp32 restatements of the same ops,
used by the tests and by the CPU execution path.
"""

from __future__ import annotations

import importlib
from typing import Optional

import torch

from . import ref  # noqa: F401

ACT = {"none": 0, None: 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1, "silu": 2, "swish": 2,
       "gelu": 3, "gelu_erf": 3}
NORM = {"rms": 0, "gemma_rms": 1, "layer": 2, "ada_rms": 3, "rms_noweight": 4}

_ext = None
ATTN_IMPL = __import__("os").environ.get("PHYAI_ATTN_IMPL", "tc")


def ext():
    """The compiled extension module; raises with build instructions if absent."""
    global _ext
    if _ext is None:
        try:
            _ext = importlib.import_module("phyai_b200._C")
        except ImportError as e:  # pragma: no cover - exercised only on a broken install
            raise RuntimeError(
                "phyai_b200._C is not built; run `python -m phyai_b200.build_ext` "
                "(needs nvcc with sm_100a support)."
            ) from e
    return _ext


def available() -> bool:
    """True when the extension is importable and a CUDA device is visible."""
    if not torch.cuda.is_available():
        return False
    try:
        ext()
    except RuntimeError:
        return False
    return True


def kernel_status() -> int:
    """Read and clear the device status word (0 = no kernel gave up on a wait)."""
    return ext().kernel_status()


def launch_counter() -> int:
    return ext().launch_counter()


def reset_launch_counter() -> None:
    ext().reset_launch_counter()


def set_pdl(on: bool) -> None:
    """Launch the library's kernels with programmatic dependent launch: a kernel's set-up
    and weight prefetch overlap the tail of its predecessor (also inside captured graphs)."""
    ext().set_pdl(bool(on))


def set_gemm_2cta(mode: int | bool | None) -> None:
    """Route large plain bf16 GEMMs to the CTA-pair kernel (``tcgen05.mma.cta_group::2``, 256 x 256
    tiles on two SMs): ``True`` / ``False``, or ``None`` to follow ``PHYAI_GEMM_2CTA``."""
    ext().set_gemm_2cta(-1 if mode is None else int(bool(mode)))


def gemm_2cta_launches() -> int:
    """How many GEMM calls the CTA-pair kernel has served in this process."""
    return int(ext().gemm_2cta_launches())


def pdl_enabled() -> bool:
    return ext().pdl_enabled()


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, *,
         bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
         res_mod: int = 0, col_gate: Optional[torch.Tensor] = None,
         row_scale: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None,
         act: str | None = "none", glu: bool = False, out_dtype: torch.dtype = torch.bfloat16,
         a_scale: Optional[torch.Tensor] = None, w_scale: Optional[torch.Tensor] = None,
         force_bn: int = 0, force_swap: int = -1, force_splits: int = 0,
         trace: Optional[torch.Tensor] = None, wait: Optional[tuple[int, int, int]] = None,
         row_rms: Optional[tuple[int, float]] = None, rope: Optional[torch.Tensor] = None,
         zero: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None,
         col_scale2: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = epilogue(x @ w.T)`` on tcgen05 tensor cores (see ``csrc/gemm.cuh``).

    ``wait=(signal_array_ptr, channel, arrivals)``: ``x`` lives in symmetric memory and is being
    written by peer GPUs; the kernel waits for that many arrivals on the channel before it loads
    ``x`` and closes the channel's call when it is done (all-gather fused into the GEMM).

    ``row_rms=(dim, eps)``: ``row_scale`` holds the sum of squares of each row of the un-normed
    activation (what another GEMM's ``sumsq`` accumulated) and the epilogue multiplies by
    ``rsqrt(row_scale / dim + eps)``: an RMSNorm whose weight was folded into ``w``.

    ``rope``: a descriptor from :func:`rope_epilogue_desc`; ``w`` is a fused QKV weight whose q / k head
    rows were permuted with :func:`permute_rope_rows`, and instead of storing ``out`` (untouched) the
    epilogue rotates q and k and writes q to its buffer and k / v to their KV-pool rows.
    ``zero``: an fp32 scratch tensor this launch clears (never one it reads or accumulates into).
    ``out2`` / ``col_scale2``: a second bf16 output ``out * (1 + col_scale2[n])`` of a plain (non-gated) store: the
    column half of an (Ada)RMS norm applied where the rows are produced; the consumer applies the row half (``row_rms``).

    ``x`` is ``(M, K)``, ``w`` is ``(N, K)`` (the ``nn.Linear`` layout), both bf16 or
    both float8_e4m3fn (then ``a_scale`` (M,) and ``w_scale`` (N,) dequantise). With
    ``glu=True`` the rows of ``w`` interleave gate and up (row ``2j`` = gate ``j``,
    row ``2j+1`` = up ``j``) and the output has ``N/2`` columns.
    """
    M, N = x.shape[0], w.shape[0]
    if out is None:
        out = torch.empty((M, N // 2 if glu else N), dtype=out_dtype, device=x.device)
    ext().gemm(x, w, out, bias, residual, res_mod, col_gate, row_scale, sumsq, ACT[act], glu,
               a_scale, w_scale, force_bn, force_swap, force_splits, trace,
               *((0, -1, 0) if wait is None else wait), *((0, 0.0) if row_rms is None else row_rms), rope, zero, out2, col_scale2)
    return out


def rope_epilogue_desc(q_out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, cos_sin: torch.Tensor,
                       pos: torch.Tensor, slots: torch.Tensor, Hq: int, Hkv: int, D: int) -> torch.Tensor:
    """Device descriptor for ``gemm(..., rope=...)``: where rotated q, k and v of a fused QKV projection go.

    Keep the descriptor and the tensors it names alive while launches (or captured graphs) use it."""
    return ext().rope_epilogue_desc(q_out, k_pool, v_pool, cos_sin, pos, slots, Hq, Hkv, D)


def permute_rope_rows(w: torch.Tensor, Hq: int, Hkv: int, D: int) -> torch.Tensor:
    """Reorder the output rows (dim 0) of a fused QKV weight or bias for the rotating epilogue: inside every
    q and k head, row ``2i`` is dimension ``i`` and row ``2i + 1`` is dimension ``i + D/2``; v rows stay."""
    half = D // 2
    idx = torch.arange(D).view(2, half).t().reshape(-1)              # 0, half, 1, half + 1, ...
    rows = torch.cat([h * D + idx for h in range(Hq + Hkv)] + [torch.arange((Hq + Hkv) * D, (Hq + 2 * Hkv) * D)])
    return w.index_select(0, rows.to(w.device)).contiguous()


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor],
              q_start: torch.Tensor, q_len: torch.Tensor, kv_indptr: torch.Tensor,
              kv_len: torch.Tensor, *, kv_indices: Optional[torch.Tensor] = None,
              max_q_len: int, causal: bool = False, splits: int = 1,
              sm_scale: Optional[float] = None, impl: Optional[str] = None,
              trace: Optional[torch.Tensor] = None, window: int = 0, soft_cap: float = 0.0) -> torch.Tensor:
    """Ragged / paged attention (see ``csrc/attention.cuh``).

    ``q`` ``(tokens, Hq, D)``; ``k``/``v`` ``(rows, Hkv, D)`` pools; sequence ``b`` owns
    query tokens ``q_start[b] + [0, q_len[b])`` and KV entries ``kv_indptr[b] +
    [0, kv_len[b])``, mapped to pool rows through ``kv_indices`` when given.
    ``impl``: ``"tc"`` (tcgen05 + tensor memory, one query tile per CTA: the latency variant),
    ``"pp"`` (tcgen05, two query tiles per CTA in ping-pong with P kept in tensor memory: the
    throughput variant for long dense sequences, head_dim <= 128) or ``"mma"`` (mma.sync). By
    default long unpaged calls take ``"pp"`` and everything else ``"tc"``.
    ``window`` > 0: a query at position ``i`` (counted from the end of its KV range) sees KV entries ``i - window + 1 .. i``
    only; ``soft_cap`` > 0: scores become ``soft_cap * tanh(score / soft_cap)`` before the softmax. Both run on ``"tc"``.
    """
    extra = window > 0 or soft_cap > 0
    if impl is None:
        impl = ATTN_IMPL
        if extra:
            impl = "tc"
        elif (impl == "tc" and max_q_len >= 512 and kv_indices is None and splits == 1 and q.shape[-1] <= 128
                and q.shape[-1] % 8 == 0):
            impl = "pp"
    if out is None:
        out = torch.empty_like(q)
    if sm_scale is None:
        sm_scale = q.shape[-1] ** -0.5
    ext().attention(q, k, v, out, q_start, q_len, kv_indptr, kv_len, kv_indices, max_q_len,
                    causal, splits, sm_scale, {"mma": 0, "tc": 1, "pp": 2}[impl], trace, int(window), float(soft_cap))
    return out


def norm(x: torch.Tensor, mode: str, *, weight: Optional[torch.Tensor] = None,
         bias: Optional[torch.Tensor] = None, mod: Optional[torch.Tensor] = None,
         group: int = 1, residual: Optional[torch.Tensor] = None,
         sumsq: Optional[torch.Tensor] = None, eps: float = 1e-6,
         out: Optional[torch.Tensor] = None, y8: Optional[torch.Tensor] = None,
         y8_scale: Optional[torch.Tensor] = None, y8_block: int = 0) -> torch.Tensor:
    """Row norms: ``rms`` / ``gemma_rms`` ((1+w)) / ``layer`` / ``ada_rms``.

    With ``residual`` the kernel first does ``residual += x`` in place and norms the
    sum. ``ada_rms`` reads ``mod`` rows ``(scale | shift | gate)`` shared by ``group``
    consecutive rows. ``y8`` additionally emits an e4m3 copy with scales.
    """
    if out is None:
        out = torch.empty_like(x)
    ext().norm(x, out, NORM[mode], weight, bias, mod, group, residual, sumsq, eps, y8, y8_scale,
               y8_block)
    return out


def rope_kv(qkv: torch.Tensor, Hq: int, Hkv: int, D: int, q_out: torch.Tensor, *,
            pos: Optional[torch.Tensor] = None, cos_sin: Optional[torch.Tensor] = None,
            rot_dim: int = 0, q_norm_w: Optional[torch.Tensor] = None,
            k_norm_w: Optional[torch.Tensor] = None, norm_eps: float = 1e-6,
            k_pool: Optional[torch.Tensor] = None, v_pool: Optional[torch.Tensor] = None,
            slots: Optional[torch.Tensor] = None, slot_base: int = 0,
            zero: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Split fused qkv rows, optional per-head RMSNorm, rotate q/k, scatter k/v to the pool.

    ``zero``: an fp32 scratch tensor the launch also clears (sum-of-squares accumulators)."""
    ext().rope_kv(qkv, Hq, Hkv, D, pos, cos_sin, rot_dim, q_norm_w, k_norm_w, norm_eps, q_out,
                  k_pool, v_pool, slots, slot_base, zero)
    return q_out


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, *, lo: int = 0,
              hi: Optional[int] = None, scale: float = 1.0,
              dst_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Masked (vocab-range) embedding lookup with scale; rows can be scattered."""
    if hi is None:
        hi = lo + table.shape[0]
    ext().embedding(ids, table, lo, hi, scale, out, dst_rows)
    return out


def im2col(pix: torch.Tensor, patch: int, out: torch.Tensor) -> torch.Tensor:
    ext().im2col(pix, patch, out)
    return out


def gdn_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
               state_pool: torch.Tensor, state_indices: torch.Tensor, *, scale: float | None = None,
               use_qk_l2norm: bool = True) -> torch.Tensor:
    """One Gated-DeltaNet decode step per sequence (``csrc/gdn.cu``): q, k ``(B, H, Dk)``, v ``(B, H, Dv)``, g, beta
    ``(B, H)``; the fp32 states ``state_pool[state_indices]`` (``(slots, H, Dk, Dv)``) are updated in place."""
    sc = q.shape[-1] ** -0.5 if scale is None else scale
    idx = state_indices.to(torch.int64).contiguous()
    return ext().gdn_decode(q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous().to(q.dtype),
                            beta.contiguous().to(q.dtype), state_pool, idx, float(sc), bool(use_qk_l2norm))


def snake(x: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """``x + sin^2(alpha x) / (beta + 1e-9)`` over ``(B, C, T)`` in one pass; ``alpha`` / ``beta`` are the
    per-channel scales (already exponentiated), any shape with C elements."""
    return ext().snake(x.contiguous(), alpha.reshape(-1).float().contiguous(), beta.reshape(-1).float().contiguous())


def gated_act(x: torch.Tensor, act: str, *, interleaved: bool = False,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty(*x.shape[:-1], x.shape[-1] // 2, dtype=x.dtype, device=x.device)
    ext().gated_act(x, out, ACT[act], interleaved)
    return out


def unary(x: torch.Tensor, act: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty_like(x)
    ext().unary(x, out, ACT[act])
    return out


def axpy(x: torch.Tensor, v: torch.Tensor, dt: float) -> torch.Tensor:
    """In place ``x += dt * v`` (the Euler flow-matching update)."""
    ext().axpy(x, v, dt)
    return x


def cfg_combine(cond: torch.Tensor, uncond: torch.Tensor, g: float, *,
                out: Optional[torch.Tensor] = None, x_fp32: Optional[torch.Tensor] = None,
                dt: float = 0.0) -> Optional[torch.Tensor]:
    """``uncond + g (cond - uncond)``, optionally fused with ``x += dt * v``."""
    if out is None and x_fp32 is None:
        out = torch.empty_like(cond)
    ext().cfg_combine(cond, uncond, g, out, x_fp32, dt)
    return out


def linear_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T + bias`` on CUDA cores with fp32 accumulation, for what :func:`gemm` does not take: fp32 / fp16
    operands, mixed operand types, K or N that is not a multiple of 8. ``x`` (M, K), ``w`` (N, K)."""
    return ext().linear_simt(x, w, bias)


def domain_linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, domain: torch.Tensor) -> torch.Tensor:
    """``x[b] @ W[domain[b]] + bias[domain[b]]`` for ``x`` (B, T, K) bf16, ``w`` (domains, K * N) in ``[K][N]`` order,
    ``bias`` (domains, N), ``domain`` int64 (B,) on the device (read by the kernel: no host synchronisation)."""
    return ext().domain_linear(x, w, bias, domain)


def unipc_step(v: torch.Tensor, x: torch.Tensor, x_last: torch.Tensor, m1: torch.Tensor, m2: torch.Tensor, *, sigma: float,
               corr: Optional[tuple], pred: tuple, v_uncond: Optional[torch.Tensor] = None, g: float = 1.0,
               keep: Optional[torch.Tensor] = None, cond: Optional[torch.Tensor] = None, view: tuple[int, int, int] | None = None,
               live_inner: int = 0) -> torch.Tensor:
    """One UniPC update of the bf16 sample ``x`` in place (guidance combine, x0 prediction, corrector, predictor,
    history rotation, clean frames re-imposed); ``x_last`` / ``m1`` / ``m2`` are fp32 state of the same size.
    ``view`` = (C, T, inner) of the ``[B, C, T, inner]`` reading that ``keep`` ``[B, T]`` and ``live_inner`` refer to."""
    C, T, inner = view if view is not None else (1, 1, x.shape[-1])
    ext().unipc_step(v, v_uncond, float(g), x, x_last, m1, m2, float(sigma), corr is not None,
                     [float(c) for c in (corr or (0.0, 0.0, 0.0, 0.0))], [float(c) for c in pred], keep, cond, C, T, inner, live_inner)
    return x


def scatter_rows(src: torch.Tensor, dst: torch.Tensor,
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    ext().scatter_rows(src, dst, rows)
    return dst


def quant_fp8(x: torch.Tensor, block: int = 0):
    """e4m3 quantisation of bf16 rows: per-row scales, or per 1x128 block (block=128)."""
    y = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    n = x.shape[1] // 128 if block else 1
    scale = torch.empty((x.shape[0], n) if block else (x.shape[0],), dtype=torch.float32,
                        device=x.device)
    ext().quant_fp8(x, y, scale, block)
    return y, scale
