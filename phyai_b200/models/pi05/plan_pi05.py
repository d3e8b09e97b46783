"""Static execution plan of Pi0.5 on B200: preallocated buffers + a fixed kernel sequence.

A request is three stages, each a straight line of this repository's sm_100a kernels
(no per-op Python dispatch, no allocation), so the whole request is captured as one
CUDA graph per prompt-length bucket:

* ``vision``  all cameras of all robots in one batch (the reference runs one robot at a
  time, phyai/src/phyai/models/pi05/scheduler_ws1_pi05.py:449-462);
* ``prefix``  18 Gemma blocks over [image | prompt] rows; K/V go straight from the epilogue
  of the QKV GEMM into the paged pool; the last block stops after its K/V write because
  nothing reads its output (the reference computes it, scheduler_ws1_pi05.py:505-511);
* ``expert``  the 10-step Euler loop, 5 kernels per block: QKV GEMM (AdaRMS row factor, RoPE and
  K/V write in its epilogue), joint attention (KV split over a cluster), o-proj GEMM with
  gated residual, sum-of-squares and the next norm's column factor in its epilogue, gate-up GEMM
  with AdaRMS row factor and GeGLU epilogue, down GEMM with gated residual, sum-of-squares and
  column-factor epilogue (the reference needs ~13, modeling_pi05.py:801-835); one copy of the
  expert weights serves every step. With ``fold_norms = False`` the unfused 8-kernel sequence
  (separate AdaRMSNorm and RoPE kernels) runs instead.

The first Euler step runs on a second stream underneath the prefix decoder (``_run_overlapped``):
block ``li`` of the expert only needs the prefix K/V of block ``li``.

KV pool layout: robot ``b`` owns the slab of slots ``1 + b*(P+C) + [0, P+C)`` (``P`` = max
prefix rows, ``C`` = chunk; slot 0 is unused padding). Its real prefix rows fill the start of
the slab and its action tokens are written directly behind them, so both the prefix
attention and the joint attention read one contiguous slot range and the attention kernel
can fetch K/V tiles with TMA instead of per-row gathers.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ... import ops
from ...cache import KVCachePool
from ...env import envs
from ...ops.expert_stack import ExpertGeometry, ExpertStack
from .modeling_pi05 import PI05Model


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class PI05Layout:
    """Host-side description of one request shape."""

    batch: int
    lang_lens: tuple[int, ...]
    lang_bucket: int


class PI05Plan:
    #: suffix tokens in front of the action tokens (Pi0 puts one state token there)
    suffix_extra = 0
    #: fold the expert's AdaRMS norms into the epilogues of the neighbouring GEMMs (one shared weight copy)
    fold_norms = True
    #: run the first Euler step on a second stream under the prefix decoder (PHYAI_PI05_OVERLAP=0 turns it off)
    overlap_first_step = bool(envs.PHYAI_PI05_OVERLAP.get())
    #: run the Euler loop as one persistent kernel (``csrc/expert_stack.cu``) where the geometry allows it; off by
    #: default: at batch 1 it measured 16.5 ms for the ten steps against 9.3 ms launch by launch
    use_expert_kernel = bool(envs.PHYAI_PI05_EXPERT_KERNEL.get())
    #: serve the prefix decoder and the action expert in block-scaled fp8 (``PHYAI_PI05_FP8=1`` or
    #: ``quantization="fp8_block"``): e4m3 weights with 128 x 128 scales, activations quantised per 1 x 128 block
    #: by the norm kernels / a quantiser in front of every GEMM; the vision tower (4304-wide MLP) stays bf16
    serve_fp8 = bool(envs.PHYAI_PI05_FP8.get())
    #: True in the subclass whose stages reduce the row-parallel products over a peer group
    tensor_parallel = False
    _side_stream = None

    def __init__(self, model: PI05Model, *, max_batch_size: int = 1, num_images: int = 3,
                 device: torch.device | str = "cuda", quantization: str | None = None) -> None:
        cfg = model.config
        self.model, self.cfg = model, cfg
        self.device = torch.device(device)
        if quantization not in (None, "bf16", "fp8_block"):
            raise ValueError(f"unknown quantization {quantization!r} (bf16 | fp8_block)")
        self.fp8 = quantization == "fp8_block" or (quantization is None and self.serve_fp8)
        if self.fp8:
            # the fp8 GEMM has no norm / rotary epilogues: the unfolded launch sequence, no second stream
            self.fold_norms, self.overlap_first_step, self.use_expert_kernel = False, False, False
        self.B, self.n_img = max_batch_size, num_images
        dt = torch.bfloat16
        if model.params_dtype != dt or model.vision.compute_dtype != dt:
            raise ValueError("PI05Plan runs bf16 weights; use the eager path for other dtypes")
        v, t, e = cfg.vision, cfg.text, cfg.expert
        # widths of this rank's slice of every projection (the whole projection on one GPU)
        lm0, ex0 = model.paligemma_lm.layers[0], model.expert_stack.layers[0]
        self.tp = int(lm0.attn.o.tp_size)
        self.Hq, self.Hkv = lm0.attn.qkv.q_size // t.head_dim, lm0.attn.qkv.kv_size // t.head_dim
        self.I_p, self.I_e = lm0.mlp.down.input_size_per_partition, ex0.mlp.down.input_size_per_partition
        # the expert may be whole on every rank while the prefix decoder is sharded (its K/V head is replicated either way)
        self.tp_e = int(ex0.attn.o.tp_size)
        self.Hq_e = ex0.attn.qkv.q_size // t.head_dim
        if ex0.attn.qkv.kv_size // t.head_dim != self.Hkv:
            raise ValueError("prefix decoder and action expert must hold the same K/V heads per rank (they share the pool)")
        if self.tp > 1 and not self.tensor_parallel:
            raise ValueError("the model is sharded over a tensor-parallel axis: build PI05TPPlan for it")
        self.img_tokens = v.num_patches * num_images
        self.P = self.img_tokens + cfg.tokenizer_max_length          # max prefix rows per robot
        self.C = cfg.chunk_size
        self.slab = self.P + self.suffix_extra + self.C
        dev = self.device
        B = self.B

        def buf(*shape, dtype=dt):
            return torch.zeros(*shape, dtype=dtype, device=dev)

        # ---------------- weights prepared for the kernels
        kp = _round_up(v.num_channels * v.patch_size ** 2, 8)
        self.patch_k = kp
        w = model.vision.patch_weight.reshape(v.hidden_size, -1)
        self.patch_w = torch.zeros(v.hidden_size, kp, dtype=dt, device=dev)
        self.patch_w[:, : w.shape[1]].copy_(w)
        self.cos_sin = model.rope.cos_sin_cache.to(dev, torch.float32).contiguous()

        # ---------------- vision buffers
        Mv = B * self.img_tokens
        self.Mv = Mv
        self.pixels = buf(B * num_images, v.num_channels, v.image_size, v.image_size)
        self.v_cols = buf(Mv, kp)
        self.v_h = buf(Mv, v.hidden_size)
        self.v_x = buf(Mv, v.hidden_size)
        self.v_qkv = buf(Mv, 3 * v.hidden_size)
        self.v_attn = buf(Mv, v.hidden_size)
        self.v_mlp = buf(Mv, v.intermediate_size)
        n_seq = B * num_images
        ar = torch.arange(n_seq, dtype=torch.int32, device=dev)
        self.v_qstart = ar * v.num_patches
        self.v_qlen = torch.full((n_seq,), v.num_patches, dtype=torch.int32, device=dev)

        # ---------------- prefix buffers (sized for the largest bucket)
        Mp = B * self.P
        H = t.hidden_size
        qkv_w = (self.Hq + 2 * self.Hkv) * t.head_dim
        self.p_h = buf(Mp, H)
        self.p_x = buf(Mp, H)
        self.p_qkv = buf(Mp, qkv_w)
        self.p_q = buf(Mp, self.Hq * t.head_dim)
        self.p_attn = buf(Mp, self.Hq * t.head_dim)
        self.p_act = buf(Mp, self.I_p)
        self.input_ids = torch.zeros(B, cfg.tokenizer_max_length, dtype=torch.int64, device=dev)
        self.pool = KVCachePool(cfg.num_layers, 1 + B * self.slab, self.Hkv, t.head_dim, dtype=dt, device=dev)
        # per-bucket metadata (filled by set_layout)
        self.p_pos = torch.zeros(Mp, dtype=torch.int32, device=dev)
        self.p_slots = torch.zeros(Mp, dtype=torch.int64, device=dev)
        self.p_qstart = torch.zeros(B, dtype=torch.int32, device=dev)
        self.p_qlen = torch.zeros(B, dtype=torch.int32, device=dev)
        self.p_kvptr = torch.zeros(B, dtype=torch.int32, device=dev)
        self.p_kvlen = torch.zeros(B, dtype=torch.int32, device=dev)
        self.lang_rows = torch.full((B * cfg.tokenizer_max_length,), -1, dtype=torch.int32, device=dev)

        # ---------------- expert buffers
        Me = B * self.C
        He = e.hidden_size
        self.Me = Me
        self.x_t = buf(Me, cfg.max_action_dim)
        self.noise = buf(B, self.C, cfg.max_action_dim)
        self.e_h = buf(Me, He)
        self.e_x = buf(Me, He)
        self.e_qkv = buf(Me, (self.Hq_e + 2 * self.Hkv) * t.head_dim)
        self.e_q = buf(Me, self.Hq_e * t.head_dim)
        self.e_attn = buf(Me, self.Hq_e * t.head_dim)
        self.e_act = buf(Me, self.I_e)
        self.e_v = buf(Me, cfg.max_action_dim)
        self.e_pos = torch.zeros(Me, dtype=torch.int32, device=dev)
        self.e_slots = torch.zeros(Me, dtype=torch.int64, device=dev)
        self.e_qstart = torch.arange(B, dtype=torch.int32, device=dev) * self.C
        self.e_qlen = torch.full((B,), self.C, dtype=torch.int32, device=dev)
        self.e_kvptr = torch.tensor([1 + b * self.slab for b in range(B)], dtype=torch.int32, device=dev)
        self.e_kvlen = torch.zeros(B, dtype=torch.int32, device=dev)
        self.out = buf(B, self.C, cfg.max_action_dim)
        if self.fp8:
            f8 = torch.float8_e4m3fn
            for name, width in (("H", H), ("Q", self.Hq * t.head_dim), ("I", self.I_p)):
                if width % 128:
                    raise ValueError(f"block-scaled fp8 needs widths that are multiples of 128, got {width}")
                setattr(self, f"p8_{name}", torch.zeros(Mp, width, dtype=f8, device=dev))
                setattr(self, f"p8s_{name}", torch.zeros(Mp, width // 128, dtype=torch.float32, device=dev))
            for name, width in (("H", He), ("Q", self.Hq_e * t.head_dim), ("I", self.I_e)):
                if width % 128:
                    raise ValueError(f"block-scaled fp8 needs widths that are multiples of 128, got {width}")
                setattr(self, f"e8_{name}", torch.zeros(Me, width, dtype=f8, device=dev))
                setattr(self, f"e8s_{name}", torch.zeros(Me, width // 128, dtype=torch.float32, device=dev))
            self.w8: dict[str, list[tuple[torch.Tensor, torch.Tensor]]] = {}
        self.mod_in: list[torch.Tensor] = []
        self.mod_post: list[torch.Tensor] = []
        self.mod_final: torch.Tensor | None = None
        self.dt = -1.0 / cfg.num_inference_steps
        # KV splits of the attention calls (a cluster of that many CTAs per head and query tile)
        self.expert_splits = int(envs.PHYAI_PI05_EXPERT_SPLITS.get() or 8)
        # batch 1: two KV splits at every prompt bucket (968 rows: 15.75 ms per request with 2, 15.90 with 4; the kernel
        # alone, inside a graph: 30.6 / 39.2 us at 968 rows, 30.2 / 38.5 us at 816)
        self._prefix_splits_env = envs.PHYAI_PI05_PREFIX_SPLITS.get()
        self.prefix_splits = int(self._prefix_splits_env or (2 if B == 1 else 1))
        self._layout_key = None
        self.stack: ExpertStack | None = None

    # ------------------------------------------------------------------ setup
    @torch.no_grad()
    def build_modulation_tables(self) -> None:
        """AdaRMS (scale|shift|gate) rows for every norm and Euler step; call after weights are loaded."""
        cfg = self.cfg
        N = cfg.num_inference_steps
        ts = 1.0 + torch.arange(N, dtype=torch.float32, device=self.device) * self.dt
        conds = self.model.heads.embed_time(ts).contiguous()
        stack = self.model.expert_stack
        self.mod_in = [l.input_layernorm.project_modulation(conds) for l in stack.layers]
        self.mod_post = [l.post_attention_layernorm.project_modulation(conds) for l in stack.layers]
        self.mod_final = stack.norm.project_modulation(conds)
        if self.fold_norms:
            self._build_expert_kernel(stack)
            self._fold_modulation(stack)
            self._fold_prefix()
        if self.fp8:
            self._build_fp8_weights(expert=True)

    def _build_fp8_weights(self, *, expert: bool) -> None:
        """Block-scaled e4m3 copies (or the stored tensors of an fp8 checkpoint) of the decoder projections."""
        from ...ops.fp8_block import layer_weight_fp8

        groups = [("p", self.model.paligemma_lm.layers)] + ([("e", self.model.expert_stack.layers)] if expert else [])
        for tag, layers in groups:
            self.w8[f"{tag}.qkv"] = [layer_weight_fp8(l.attn.qkv) for l in layers]
            self.w8[f"{tag}.o"] = [layer_weight_fp8(l.attn.o) for l in layers]
            self.w8[f"{tag}.gate_up"] = [layer_weight_fp8(l.mlp.gate_up) for l in layers]
            self.w8[f"{tag}.down"] = [layer_weight_fp8(l.mlp.down) for l in layers]

    def _expert_geometry(self) -> ExpertGeometry:
        cfg, e, t = self.cfg, self.cfg.expert, self.cfg.text
        return ExpertGeometry(rows=self.Me, hidden=e.hidden_size, inter=e.intermediate_size, q_heads=self.Hq_e,
                              head_dim=t.head_dim, action_dim=cfg.max_action_dim, layers=cfg.num_layers,
                              steps=cfg.num_inference_steps)

    def _build_expert_kernel(self, stack) -> None:
        """Tables of the persistent expert kernel: the AdaRMS modulation of every (step, block) as fp32
        column factors, branch gates and ``shift @ W^T`` biases; the weights stay as loaded (one copy)."""
        self.stack = None
        t = self.cfg.text
        if not (self.use_expert_kernel and self.device.type == "cuda" and self.B == 1 and t.num_key_value_heads == 1 and self.tp_e == 1
                and self.suffix_extra == 0):
            return
        geo = self._expert_geometry()
        if not ExpertStack.supports(geo, self.slab):
            return
        He, heads = geo.hidden, self.model.heads
        st = ExpertStack(geo, device=self.device)
        st.set_weights([(l.attn.qkv.weight, l.attn.o.weight, l.mlp.gate_up.weight, l.mlp.down.weight) for l in stack.layers])

        def cols(mods, a, b):          # [layers][steps, 3He] -> [steps, layers, He]
            return torch.stack([m[:, a:b].float() for m in mods], dim=1)

        def biases(mods, weights):     # shift @ W^T -> [steps, layers, N]
            return torch.stack([m[:, He:2 * He].float() @ w.float().t() for m, w in zip(mods, weights)], dim=1)

        st.set_tables(in_scale=1.0 + cols(self.mod_in, 0, He), post_scale=1.0 + cols(self.mod_post, 0, He),
                      gate_in=cols(self.mod_in, 2 * He, 3 * He), gate_post=cols(self.mod_post, 2 * He, 3 * He),
                      qkv_bias=biases(self.mod_in, [l.attn.qkv.weight for l in stack.layers]),
                      gu_bias=biases(self.mod_post, [l.mlp.gate_up.weight for l in stack.layers]),
                      fin_scale=1.0 + self.mod_final[:, :He].float(),
                      out_bias=self.mod_final[:, He:2 * He].float() @ heads.action_out_proj.weight.float().t()
                      + heads.action_out_proj.bias.float()[None, :])
        self.stack = st

    def _run_expert_kernel(self, step_begin: int, step_end: int) -> None:
        cfg, e, t, heads = self.cfg, self.cfg.expert, self.cfg.text, self.model.heads
        self.stack.run(w_in=heads.action_in_proj.weight, b_in=heads.action_in_proj.bias, w_out=heads.action_out_proj.weight,
                       k_pool=self.pool.k, v_pool=self.pool.v, kv_ptr=self.e_kvptr, kv_len=self.e_kvlen, pos=self.e_pos,
                       cos_sin=self.cos_sin, x0=self.x_t, out=self.x_t, eps=e.rms_norm_eps, dt=self.dt,
                       sm_scale=t.head_dim ** -0.5, step_begin=step_begin, step_end=step_end)

    def _fold_prefix(self) -> None:
        """Prefix decoder: Gemma RMSNorm weights (1 + w) folded into the QKV and gate/up weights (one
        static copy each), QKV rows reordered for the rotating epilogue; block 0 keeps its norm kernel."""
        t, lm = self.cfg.text, self.model.paligemma_lm
        Hq, Hkv, D = self.Hq, self.Hkv, t.head_dim

        def fold(w, norm_w):
            return (w.float() * (1.0 + norm_w.float())[None, :]).to(torch.bfloat16).contiguous()

        self.pfold_qkv = [ops.permute_rope_rows(fold(l.attn.qkv.weight, l.input_layernorm.weight) if li > 0
                                                else l.attn.qkv.weight, Hq, Hkv, D) for li, l in enumerate(lm.layers)]
        self.pfold_gate_up = [fold(l.mlp.gate_up.weight, l.post_attention_layernorm.weight) for l in lm.layers[:-1]]
        self.p_rope = self._rope_descs(self.p_q, self.p_pos, self.p_slots)
        self.p_ss = torch.zeros(2, self.B * self.P, dtype=torch.float32, device=self.device)

    def _fold_modulation(self, stack) -> None:
        """AdaRMS without a norm kernel and with ONE copy of the weights: ``norm(h) @ W^T`` is evaluated as
        ``((h * (1 + scale)) @ W^T) * rsqrt(mean(h^2) + eps) + shift @ W^T``. The column factor is applied by the
        epilogue of the GEMM that produces ``h`` (its second output, ``out2``), together with the row sums of squares;
        the row factor by the epilogue of the consuming GEMM; ``shift @ W^T`` is a bias row per Euler step (kilobytes)."""
        He = self.cfg.expert.hidden_size
        dt = torch.bfloat16

        def shift_bias(w: torch.Tensor, mod: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
            b = mod[:, He:2 * He].float() @ w.float().T                      # (steps, N)
            if bias is not None:
                b = b + bias.float()[None, :]
            return b.to(dt).contiguous()

        t = self.cfg.text
        Hq, Hkv, D = self.Hq_e, self.Hkv, t.head_dim
        self.folded_steps = self.cfg.num_inference_steps
        self.fold_qkv, self.fold_gate_up = [], []
        for li, layer in enumerate(stack.layers):
            # q / k head rows reordered for the rotating epilogue of the QKV GEMM. The first block of a
            # step keeps its norm kernel (nothing upstream produces its scaled rows): no bias.
            wq = ops.permute_rope_rows(layer.attn.qkv.weight, Hq, Hkv, D)
            self.fold_qkv.append((wq, shift_bias(wq, self.mod_in[li]) if li > 0 else None))
            self.fold_gate_up.append((layer.mlp.gate_up.weight, shift_bias(layer.mlp.gate_up.weight, self.mod_post[li])))
        self.rope_desc = self._rope_descs(self.e_q, self.e_pos, self.e_slots, self.Hq_e)
        heads = self.model.heads
        self.fold_out = (heads.action_out_proj.weight, shift_bias(heads.action_out_proj.weight, self.mod_final, heads.action_out_proj.bias))
        self.e_ss = torch.zeros(2, self.Me, dtype=torch.float32, device=self.device)
        self.e_x2 = torch.zeros(self.Me, He, dtype=dt, device=self.device)      # h * (1 + scale) of the norm that comes next

    def _rope_descs(self, q_out: torch.Tensor, pos: torch.Tensor, slots: torch.Tensor, q_heads: int | None = None) -> list[torch.Tensor]:
        """One rotate-and-scatter destination per layer (its K/V pool) for the QKV GEMM epilogue."""
        t = self.cfg.text
        Hq = self.Hq if q_heads is None else q_heads
        return [ops.rope_epilogue_desc(q_out, *self.pool.layer(li), self.cos_sin, pos, slots, Hq, self.Hkv, t.head_dim) for li in range(self.cfg.num_layers)]

    def set_layout(self, layout: PI05Layout) -> bool:
        """Write the metadata of a request shape into the static buffers. Returns True if it changed."""
        key = (layout.batch, layout.lang_lens, layout.lang_bucket)
        if key == self._layout_key:
            return False
        cfg, B, dev = self.cfg, self.B, self.device
        n_per = self.img_tokens + layout.lang_bucket
        real = [self.img_tokens + l for l in layout.lang_lens] + [0] * (B - layout.batch)
        base = [1 + b * self.slab for b in range(B)]
        j = torch.arange(n_per, dtype=torch.int64)
        pos = j.repeat(B)
        slots = torch.cat([base[b] + j for b in range(B)])
        Mp = B * n_per
        self.p_pos[:Mp].copy_(pos.to(torch.int32))
        self.p_slots[:Mp].copy_(slots)
        self.p_qstart.copy_(torch.arange(B, dtype=torch.int32) * n_per)
        self.p_qlen.fill_(n_per)
        self.p_kvptr.copy_(torch.tensor(base, dtype=torch.int32))
        self.p_kvlen.copy_(torch.tensor(real, dtype=torch.int32))
        L = cfg.tokenizer_max_length
        rows = torch.full((B, L), -1, dtype=torch.int32)
        for b in range(B):
            rows[b, : layout.lang_bucket] = b * n_per + self.img_tokens + torch.arange(layout.lang_bucket, dtype=torch.int32)
        self.lang_rows.copy_(rows.flatten())
        c = torch.arange(self.C, dtype=torch.int64)
        x = self.suffix_extra
        self.e_pos.copy_(torch.cat([real[b] + x + c for b in range(B)]).to(torch.int32))
        self.e_slots.copy_(torch.cat([base[b] + real[b] + x + c for b in range(B)]))
        self.e_kvlen.copy_(torch.tensor([r + x + self.C for r in real], dtype=torch.int32))
        self._real, self._base = real, base
        self._layout_key = key
        return True

    # ----------------------------------------------------------------- stages
    def vision(self, img_lo: int = 0, img_hi: int | None = None) -> None:
        """Cameras ``[img_lo, img_hi)`` of the batch (all of them by default) through the tower; their rows
        land at the start of ``v_x``."""
        cfg, v, m = self.cfg, self.cfg.vision, self.model.vision
        hi = self.B * self.n_img if img_hi is None else img_hi
        n = hi - img_lo
        if n <= 0:
            return
        M = n * v.num_patches
        cols, h, x, qkv, attn, mlp = (b[:M] for b in (self.v_cols, self.v_h, self.v_x, self.v_qkv, self.v_attn, self.v_mlp))
        qstart, qlen = self.v_qstart[:n], self.v_qlen[:n]
        ops.im2col(self.pixels[img_lo:hi], v.patch_size, cols)
        ops.gemm(cols, self.patch_w, h, bias=m.patch_bias, residual=m.position_embedding, res_mod=v.num_patches)
        H, hd, nh = v.hidden_size, v.head_dim, v.num_attention_heads
        q3 = qkv[:, :H].unflatten(1, (nh, hd))
        k3 = qkv[:, H:2 * H].unflatten(1, (nh, hd))
        v3 = qkv[:, 2 * H:].unflatten(1, (nh, hd))
        a3 = attn.unflatten(1, (nh, hd))
        for blk in m.blocks:
            ops.norm(h, "layer", weight=blk.ln1.weight, bias=blk.ln1.bias, eps=v.layer_norm_eps, out=x)
            ops.gemm(x, blk.qkv.weight, qkv, bias=blk.qkv.bias)
            ops.attention(q3, k3, v3, a3, qstart, qlen, qstart, qlen, max_q_len=v.num_patches, sm_scale=hd ** -0.5)
            ops.gemm(attn, blk.out.weight, h, bias=blk.out.bias, residual=h)
            ops.norm(h, "layer", weight=blk.ln2.weight, bias=blk.ln2.bias, eps=v.layer_norm_eps, out=x)
            ops.gemm(x, blk.fc1.weight, mlp, bias=blk.fc1.bias, act="gelu_tanh")
            ops.gemm(mlp, blk.fc2.weight, h, bias=blk.fc2.bias, residual=h)
        ops.norm(h, "layer", weight=m.post_layernorm.weight, bias=m.post_layernorm.bias, eps=v.layer_norm_eps, out=x)

    def prefix(self, lang_bucket: int, kv_events=None) -> None:
        cfg, t, lm = self.cfg, self.cfg.text, self.model.paligemma_lm
        n_per = self.img_tokens + lang_bucket
        Mp = self.B * n_per
        h, x = self.p_h[:Mp], self.p_x[:Mp]
        # image rows: projector output lands directly in the packed prefix rows of each robot
        proj = self.model.vision.projector
        for b in range(self.B):
            ops.gemm(self.v_x[b * self.img_tokens:(b + 1) * self.img_tokens], proj.weight,
                     h[b * n_per: b * n_per + self.img_tokens], bias=proj.bias)
        ops.embedding(self.input_ids.view(-1), lm.embed_tokens, h, scale=lm.embed_scale, dst_rows=self.lang_rows)
        Hq, Hkv, D = self.Hq, self.Hkv, t.head_dim
        qkv, q, attn, act = self.p_qkv[:Mp], self.p_q[:Mp], self.p_attn[:Mp], self.p_act[:Mp]
        q3, a3 = q.unflatten(1, (Hq, D)), attn.unflatten(1, (Hq, D))
        last = len(lm.layers) - 1
        if self.fold_norms:
            # five launches per block: norms, rotary embedding and the K/V scatter live in GEMM epilogues
            ss_in, ss_post = self.p_ss[0], self.p_ss[1]
            rms = (t.hidden_size, t.rms_norm_eps)
            for li, layer in enumerate(lm.layers):
                kpool, vpool = self.pool.layer(li)
                if li == 0:
                    ops.norm(h, "gemma_rms", weight=layer.input_layernorm.weight, eps=t.rms_norm_eps, out=x)
                    ops.gemm(x, self.pfold_qkv[li], qkv, rope=self.p_rope[li])
                else:
                    ops.gemm(h, self.pfold_qkv[li], qkv, row_scale=ss_in, row_rms=rms, rope=self.p_rope[li])
                if kv_events is not None:
                    kv_events[li].record(torch.cuda.current_stream())     # this block's prefix K / V are in the pool
                if li == last:
                    break  # only this block's K/V are consumed downstream
                ops.attention(q3, kpool, vpool, a3, self.p_qstart, self.p_qlen, self.p_kvptr, self.p_kvlen,
                              max_q_len=n_per, splits=self.prefix_splits, sm_scale=D ** -0.5)
                ops.gemm(attn, layer.attn.o.weight, h, residual=h, sumsq=ss_post, zero=ss_in)
                ops.gemm(h, self.pfold_gate_up[li], act, row_scale=ss_post, row_rms=rms, act="gelu_tanh", glu=True)
                ops.gemm(act, layer.mlp.down.weight, h, residual=h, sumsq=ss_in, zero=ss_post)
            return
        if self.fp8:
            from ...ops.fp8_block import gemm_fp8_block as g8, quantize_rows_into as q8

            x8, xs = self.p8_H[:Mp], self.p8s_H[:Mp]
            a8, as_ = self.p8_Q[:Mp], self.p8s_Q[:Mp]
            m8, ms = self.p8_I[:Mp], self.p8s_I[:Mp]
            W = self.w8
            for li, layer in enumerate(lm.layers):
                kpool, vpool = self.pool.layer(li)
                ops.norm(h, "gemma_rms", weight=layer.input_layernorm.weight, eps=t.rms_norm_eps, out=x, y8=x8, y8_scale=xs, y8_block=128)
                g8(x8, xs, *W["p.qkv"][li], qkv)
                ops.rope_kv(qkv, Hq, Hkv, D, q, pos=self.p_pos[:Mp], cos_sin=self.cos_sin, k_pool=kpool, v_pool=vpool,
                            slots=self.p_slots[:Mp])
                if kv_events is not None:
                    kv_events[li].record(torch.cuda.current_stream())
                if li == last:
                    break
                ops.attention(q3, kpool, vpool, a3, self.p_qstart, self.p_qlen, self.p_kvptr, self.p_kvlen,
                              max_q_len=n_per, splits=self.prefix_splits, sm_scale=D ** -0.5)
                q8(attn, a8, as_)
                g8(a8, as_, *W["p.o"][li], h, residual=h)
                ops.norm(h, "gemma_rms", weight=layer.post_attention_layernorm.weight, eps=t.rms_norm_eps, out=x, y8=x8, y8_scale=xs,
                         y8_block=128)
                g8(x8, xs, *W["p.gate_up"][li], act, act="gelu_tanh", glu=True)
                q8(act, m8, ms)
                g8(m8, ms, *W["p.down"][li], h, residual=h)
            return
        for li, layer in enumerate(lm.layers):
            kpool, vpool = self.pool.layer(li)
            ops.norm(h, "gemma_rms", weight=layer.input_layernorm.weight, eps=t.rms_norm_eps, out=x)
            ops.gemm(x, layer.attn.qkv.weight, qkv)
            ops.rope_kv(qkv, Hq, Hkv, D, q, pos=self.p_pos[:Mp], cos_sin=self.cos_sin, k_pool=kpool, v_pool=vpool,
                        slots=self.p_slots[:Mp])
            if li == last:
                break  # only this block's K/V are consumed downstream
            ops.attention(q3, kpool, vpool, a3, self.p_qstart, self.p_qlen, self.p_kvptr, self.p_kvlen,
                          max_q_len=n_per, splits=self.prefix_splits, sm_scale=D ** -0.5)
            ops.gemm(attn, layer.attn.o.weight, h, residual=h)
            ops.norm(h, "gemma_rms", weight=layer.post_attention_layernorm.weight, eps=t.rms_norm_eps, out=x)
            ops.gemm(x, layer.mlp.gate_up.weight, act, act="gelu_tanh", glu=True)
            ops.gemm(act, layer.mlp.down.weight, h, residual=h)

    def expert(self) -> None:
        cfg, e, t = self.cfg, self.cfg.expert, self.cfg.text
        heads, stack = self.model.heads, self.model.expert_stack
        Hq, Hkv, D, He, Me = self.Hq_e, self.Hkv, t.head_dim, e.hidden_size, self.Me
        h, x = self.e_h, self.e_x
        q3, a3 = self.e_q.unflatten(1, (Hq, D)), self.e_attn.unflatten(1, (Hq, D))
        self.x_t.copy_(self.noise.view(Me, -1))
        if self.fold_norms:
            return self._expert_folded()
        if self.fp8:
            return self._expert_fp8()
        for i in range(cfg.num_inference_steps):
            ops.gemm(self.x_t, heads.action_in_proj.weight, h, bias=heads.action_in_proj.bias)
            for li, layer in enumerate(stack.layers):
                kpool, vpool = self.pool.layer(li)
                m_in, m_post = self.mod_in[li][i:i + 1], self.mod_post[li][i:i + 1]
                ops.norm(h, "ada_rms", mod=m_in, group=Me, eps=e.rms_norm_eps, out=x)
                ops.gemm(x, layer.attn.qkv.weight, self.e_qkv)
                ops.rope_kv(self.e_qkv, Hq, Hkv, D, self.e_q, pos=self.e_pos, cos_sin=self.cos_sin, k_pool=kpool,
                            v_pool=vpool, slots=self.e_slots)
                ops.attention(q3, kpool, vpool, a3, self.e_qstart, self.e_qlen, self.e_kvptr, self.e_kvlen,
                              max_q_len=self.C, splits=self.expert_splits, sm_scale=D ** -0.5)
                ops.gemm(self.e_attn, layer.attn.o.weight, h, residual=h, col_gate=m_in[0, 2 * He:])
                ops.norm(h, "ada_rms", mod=m_post, group=Me, eps=e.rms_norm_eps, out=x)
                ops.gemm(x, layer.mlp.gate_up.weight, self.e_act, act="gelu_tanh", glu=True)
                ops.gemm(self.e_act, layer.mlp.down.weight, h, residual=h, col_gate=m_post[0, 2 * He:])
            ops.norm(h, "ada_rms", mod=self.mod_final[i:i + 1], group=Me, eps=e.rms_norm_eps, out=x)
            ops.gemm(x, heads.action_out_proj.weight, self.e_v, bias=heads.action_out_proj.bias)
            ops.axpy(self.x_t, self.e_v, self.dt)
        self.out.view(Me, -1).copy_(self.x_t)

    def _expert_fp8(self) -> None:
        """The Euler loop with block-scaled fp8 projections: the AdaRMS kernels emit the e4m3 rows and their
        1 x 128 scales directly, attention output and the GeGLU product pass through the quantiser; gates and
        residual adds stay in the GEMM epilogues. Ten launches per block."""
        from ...ops.fp8_block import gemm_fp8_block as g8, quantize_rows_into as q8

        cfg, e, t = self.cfg, self.cfg.expert, self.cfg.text
        heads, stack = self.model.heads, self.model.expert_stack
        Hq, Hkv, D, He, Me = self.Hq_e, self.Hkv, t.head_dim, e.hidden_size, self.Me
        h, x, W = self.e_h, self.e_x, self.w8
        q3, a3 = self.e_q.unflatten(1, (Hq, D)), self.e_attn.unflatten(1, (Hq, D))
        x8, xs, a8, as_, m8, ms = self.e8_H, self.e8s_H, self.e8_Q, self.e8s_Q, self.e8_I, self.e8s_I
        for i in range(cfg.num_inference_steps):
            ops.gemm(self.x_t, heads.action_in_proj.weight, h, bias=heads.action_in_proj.bias)
            for li, layer in enumerate(stack.layers):
                kpool, vpool = self.pool.layer(li)
                m_in, m_post = self.mod_in[li][i:i + 1], self.mod_post[li][i:i + 1]
                ops.norm(h, "ada_rms", mod=m_in, group=Me, eps=e.rms_norm_eps, out=x, y8=x8, y8_scale=xs, y8_block=128)
                g8(x8, xs, *W["e.qkv"][li], self.e_qkv)
                ops.rope_kv(self.e_qkv, Hq, Hkv, D, self.e_q, pos=self.e_pos, cos_sin=self.cos_sin, k_pool=kpool,
                            v_pool=vpool, slots=self.e_slots)
                ops.attention(q3, kpool, vpool, a3, self.e_qstart, self.e_qlen, self.e_kvptr, self.e_kvlen,
                              max_q_len=self.C, splits=self.expert_splits, sm_scale=D ** -0.5)
                q8(self.e_attn, a8, as_)
                g8(a8, as_, *W["e.o"][li], h, residual=h, col_gate=m_in[0, 2 * He:])
                ops.norm(h, "ada_rms", mod=m_post, group=Me, eps=e.rms_norm_eps, out=x, y8=x8, y8_scale=xs, y8_block=128)
                g8(x8, xs, *W["e.gate_up"][li], self.e_act, act="gelu_tanh", glu=True)
                q8(self.e_act, m8, ms)
                g8(m8, ms, *W["e.down"][li], h, residual=h, col_gate=m_post[0, 2 * He:])
            ops.norm(h, "ada_rms", mod=self.mod_final[i:i + 1], group=Me, eps=e.rms_norm_eps, out=x)
            ops.gemm(x, heads.action_out_proj.weight, self.e_v, bias=heads.action_out_proj.bias)
            ops.axpy(self.x_t, self.e_v, self.dt)
        self.out.view(Me, -1).copy_(self.x_t)

    def _expert_folded(self, steps=None, before_block=None, finish: bool = True) -> None:
        """Five launches per block: the two AdaRMS kernels live in the GEMM epilogues around them, rotary
        embedding and the K/V scatter in the epilogue of the QKV GEMM. ``steps``: which Euler steps to issue
        (default all); ``before_block(li)`` runs before block ``li`` is issued (the overlapped schedule waits
        there for the prefix K/V of that block: the wait has to precede this block's own K/V scatter, because
        the padded prompt rows of the prefix land in the pool slots the action tokens use); ``finish`` copies
        the result out."""
        cfg, e, t = self.cfg, self.cfg.expert, self.cfg.text
        heads, stack = self.model.heads, self.model.expert_stack
        Hq, Hkv, D, He, Me = self.Hq_e, self.Hkv, t.head_dim, e.hidden_size, self.Me
        h, x = self.e_h, self.e_x
        q3, a3 = self.e_q.unflatten(1, (Hq, D)), self.e_attn.unflatten(1, (Hq, D))
        ss_in, ss_post = self.e_ss[0], self.e_ss[1]
        rms = (He, e.rms_norm_eps)
        steps = list(range(cfg.num_inference_steps) if steps is None else steps)
        if self.stack is not None and before_block is None and steps:
            # the whole range in one persistent launch (the per-block hook needs launch boundaries)
            if steps != list(range(steps[0], steps[-1] + 1)):
                raise ValueError("the persistent expert kernel runs a contiguous range of Euler steps")
            self._run_expert_kernel(steps[0], steps[-1] + 1)
            steps = []
        x2, n_layers = self.e_x2, len(stack.layers)
        for i in steps:
            if i >= self.folded_steps:
                raise RuntimeError(f"Euler step {i} has no folded biases (only {self.folded_steps} kept)")
            ops.gemm(self.x_t, heads.action_in_proj.weight, h, bias=heads.action_in_proj.bias)
            for li, layer in enumerate(stack.layers):
                kpool, vpool = self.pool.layer(li)
                m_in, m_post = self.mod_in[li][i:i + 1], self.mod_post[li][i:i + 1]
                nxt = self.mod_in[li + 1][i] if li + 1 < n_layers else self.mod_final[i]
                if before_block is not None:
                    before_block(li)
                # the QKV epilogue rotates q / k and writes k / v into this block's pool rows
                w, b = self.fold_qkv[li]
                if li == 0:
                    ops.norm(h, "ada_rms", mod=m_in, group=Me, eps=e.rms_norm_eps, out=x)
                    ops.gemm(x, w, self.e_qkv, rope=self.rope_desc[li])
                else:
                    ops.gemm(x2, w, self.e_qkv, bias=b[i], row_scale=ss_in, row_rms=rms, rope=self.rope_desc[li])
                ops.attention(q3, kpool, vpool, a3, self.e_qstart, self.e_qlen, self.e_kvptr, self.e_kvlen,
                              max_q_len=self.C, splits=self.expert_splits, sm_scale=D ** -0.5)
                # each accumulating GEMM clears the other accumulator, which is idle at that point, and leaves the rows
                # scaled by the next norm's column factor beside the residual stream
                ops.gemm(self.e_attn, layer.attn.o.weight, h, residual=h, col_gate=m_in[0, 2 * He:], sumsq=ss_post,
                         zero=ss_in, out2=x2, col_scale2=m_post[0, :He])
                w, b = self.fold_gate_up[li]
                ops.gemm(x2, w, self.e_act, bias=b[i], row_scale=ss_post, row_rms=rms, act="gelu_tanh", glu=True)
                ops.gemm(self.e_act, layer.mlp.down.weight, h, residual=h, col_gate=m_post[0, 2 * He:], sumsq=ss_in,
                         zero=ss_post, out2=x2, col_scale2=nxt[:He])
            w, b = self.fold_out
            ops.gemm(x2, w, self.e_v, bias=b[i], row_scale=ss_in, row_rms=rms)
            ops.axpy(self.x_t, self.e_v, self.dt)
        if finish:
            self.out.view(Me, -1).copy_(self.x_t)

    def run(self, lang_bucket: int) -> torch.Tensor:
        """The whole request; inputs are ``pixels``, ``input_ids``, ``noise``; result in ``out``."""
        if self.overlap_first_step and self.fold_norms and self._first_step_overlappable() and self.device.type == "cuda":
            return self._run_overlapped(lang_bucket)
        self.encode_images()
        self.prefix(lang_bucket)
        self.expert()
        return self.out

    def encode_images(self) -> None:
        """Everything in front of the prefix decoder (a tensor-parallel plan splits the cameras over its ranks here)."""
        self.vision()

    def _first_step_overlappable(self) -> bool:
        """Whether ``_expert_folded(steps=[0])`` is this plan's first Euler step (subclasses with their own expert say no)."""
        return type(self).expert is PI05Plan.expert

    def _run_overlapped(self, lang_bucket: int) -> torch.Tensor:
        """Same request with the first Euler step on a second stream. Block ``li`` of the expert only needs
        the prefix K/V of block ``li``, so the first step (launch-bound, a few CTAs per kernel) runs under the
        compute-bound prefix decoder: it waits, block by block, on an event recorded after the prefix QKV
        GEMM that wrote that block's K/V. The streams join before the second step. Works eagerly and inside
        a stream capture (the event edges become graph dependencies)."""
        main = torch.cuda.current_stream()
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device)
        side = self._side_stream
        n_layers = self.cfg.num_layers
        fork, join = torch.cuda.Event(), torch.cuda.Event()
        kv_ready = [torch.cuda.Event() for _ in range(n_layers)]
        fork.record(main)
        self.encode_images()
        self.prefix(lang_bucket, kv_events=kv_ready)
        with torch.cuda.stream(side):
            side.wait_event(fork)
            self.x_t.copy_(self.noise.view(self.Me, -1))
            self._expert_folded(steps=[0], before_block=lambda li: side.wait_event(kv_ready[li]), finish=False)
            join.record(side)
        main.wait_event(join)
        self._expert_folded(steps=range(1, self.cfg.num_inference_steps))
        return self.out


__all__ = ["PI05Plan", "PI05Layout"]
