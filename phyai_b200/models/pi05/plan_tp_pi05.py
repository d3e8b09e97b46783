"""Tensor-parallel execution plan of Pi0.5: the single-GPU plan with every row-parallel product
leaving its GEMM through the epilogue into the peers' memory.

Sharding (the model's parallel linear layers decide it): q heads and MLP columns are split over the
``tp`` ranks, the single K/V head is replicated, so every rank keeps the whole K/V pool and runs
attention on its own heads only. Per block and rank that leaves two partial products (o-proj, down).
Each one is ONE GEMM whose epilogue stores the partial tile into a slot of every rank's symmetric
buffer, followed by ONE kernel that waits for the peers' tiles, sums them, applies the gate and the
residual, and writes the *next* norm of the block (Gemma RMS in the prefix decoder, AdaRMS with that
step's modulation row in the action expert) -- no all-reduce launch, no separate norm launch, no
separate rotary launch (the QKV epilogue rotates and scatters K/V as on one GPU). Seven launches per
block against the reference layer's thirteen plus two NCCL all-reduces
(phyai/src/phyai/layers/linear/layers.py:602-631, phyai/src/phyai/models/pi05/modeling_pi05.py:504-523, :801-835).

The vision tower is not sharded: 72-wide heads and a 4304-wide MLP split badly, and the cameras are
independent, so each rank encodes ``ceil(cameras / tp)`` of them with whole weights and the projected
rows are exchanged once (a peer-memory all-gather of 256 x 2048 rows per camera).

The action expert (0.6 GB) is normally kept whole on every rank (``expert_axis=None`` on the model): each rank then runs
the ten Euler steps of the single-GPU plan on its own copy of the K/V pool with no communication at all, first step
under the prefix decoder on a second stream, and tensor parallelism shortens what is big (the 2 B-parameter prefix
decoder, the cameras) without taxing what is latency-bound. A sharded expert is served too (two fused reductions per
block, AdaRMS applied by the reducing kernel).

Every rank must be given the same request; all ranks finish with bit-identical action chunks (each sums
the partials in rank order). The request is captured as one CUDA graph per prompt bucket like the
single-GPU plan; waits on peers are bounded, so ranks have to enter a replay within a second of each other.
"""

from __future__ import annotations

import torch

from ... import ops
from ... import parallel as P
from ...env import envs
from .modeling_pi05 import PI05Model
from .plan_pi05 import PI05Plan


def split_cameras(n_cameras: int, world: int, rank: int) -> tuple[int, int, int]:
    """``(per_rank, first, last)``: contiguous blocks of ``ceil(n / world)`` cameras per rank, in rank order, so that the
    all-gather of equally sized (padded) blocks returns the cameras in their original order; ranks past the end get
    an empty range."""
    per = -(-n_cameras // world)
    lo = min(rank * per, n_cameras)
    return per, lo, min(lo + per, n_cameras)


class PI05TPPlan(PI05Plan):
    tensor_parallel = True
    use_expert_kernel = False
    #: prefix reductions switch from "push the whole partial" to scatter / gather at this many rows (groups of 4+)
    scatter_min_rows = int(envs.PHYAI_PI05_TP_SCATTER_ROWS.get())

    def __init__(self, model: PI05Model, *, max_batch_size: int = 1, num_images: int = 3, device="cuda",
                 quantization: str | None = None, axis: str = "tp", mesh=None) -> None:
        if quantization not in (None, "bf16"):
            raise ValueError("the tensor-parallel plan serves bf16 (the epilogue that stores into peer memory is the bf16 GEMM's)")
        super().__init__(model, max_batch_size=max_batch_size, num_images=num_images, device=device, quantization="bf16")
        self.axis = axis
        self.mesh = mesh if mesh is not None else P.default_mesh()
        # a whole expert on every rank runs the single-GPU Euler loop (folded norms, first step on the second stream);
        # a sharded one reduces over the same signal channel as the prefix decoder, so it cannot run beside it
        self.expert_replicated = self.tp_e == 1
        self.fold_norms = self.expert_replicated
        self.overlap_first_step = self.expert_replicated and type(self).overlap_first_step
        self.rank = int(model.paligemma_lm.layers[0].attn.o.tp_rank)
        cfg, v, t = self.cfg, self.cfg.vision, self.cfg.text
        n_all = self.B * self.n_img
        if self.tp < 2:
            raise ValueError("a single rank: build PI05Plan")
        if model.vision.axis is not None and model.vision.blocks[0].out.tp_size > 1:
            raise ValueError("build the model with vision_axis=None: this plan splits the cameras, not the vision weights")
        if cfg.expert.hidden_size > t.hidden_size:
            raise ValueError("slot width is the prefix decoder's hidden size")
        from ...parallel.symm import PeerGroup

        H = t.hidden_size
        rows = max(self.B * self.P, self.Me)
        self.per, self.img_lo, self.img_hi = split_cameras(n_all, self.tp, self.rank)
        img_rows = self.per * v.num_patches
        # prefix rows at or above the threshold go reduce-scatter -> norm -> all-gather (each rank sums and norms
        # only the rows it owns and every wire carries 1 / tp of the matrix twice, instead of the whole partial
        # to every peer); the 50-row expert calls always push the whole partial
        p_rows = self.B * self.P
        self.scatter = self.tp >= 4 and p_rows >= self.scatter_min_rows
        per = -(-p_rows // self.tp)
        need = 2 * self.tp * (rows + img_rows + (per if self.scatter else 0)) * H * 2 + p_rows * H * 2 + (8 << 20)
        pg = PeerGroup.for_axis(self.mesh, axis, heap_bytes=max(need, 256 << 20))
        self.pg = pg
        self.st = pg.stream(f"pi05.tp:{rows}", rows, H)
        self.st_sc = pg.stream(f"pi05.tp.sc:{p_rows}", per, H, gather_rows=p_rows, gather_cols=H) if self.scatter else None
        self.st_img = pg.stream(f"pi05.tp.img:{img_rows}", img_rows, H)
        self.v_proj = torch.zeros(img_rows, H, dtype=torch.bfloat16, device=self.device)
        self.v_all = torch.zeros(self.tp * img_rows, H, dtype=torch.bfloat16, device=self.device)

    @torch.no_grad()
    def build_modulation_tables(self) -> None:
        super().build_modulation_tables()
        t = self.cfg.text
        Hq, Hkv, D = self.Hq, self.Hkv, t.head_dim
        # q / k rows of this rank's QKV slice reordered for the rotating epilogue
        self.tp_pqkv = [ops.permute_rope_rows(l.attn.qkv.weight, Hq, Hkv, D) for l in self.model.paligemma_lm.layers]
        self.p_rope = self._rope_descs(self.p_q, self.p_pos, self.p_slots)
        if not self.expert_replicated:
            self.tp_eqkv = [ops.permute_rope_rows(l.attn.qkv.weight, self.Hq_e, Hkv, D) for l in self.model.expert_stack.layers]
            self.rope_desc = self._rope_descs(self.e_q, self.e_pos, self.e_slots, self.Hq_e)
        for m in (*self.mod_in, *self.mod_post, self.mod_final):
            if m.dtype != torch.bfloat16 or not m.is_contiguous():
                raise ValueError("modulation rows must be contiguous bf16 for the reduce kernel")

    def _fold_prefix(self) -> None:
        """Nothing to fold: the reducing kernel of the previous product applies each prefix norm."""

    def _first_step_overlappable(self) -> bool:
        return self.expert_replicated

    def encode_images(self) -> None:
        self.images()

    # ----------------------------------------------------------------- stages
    def _reduce(self, x_part: torch.Tensor, w: torch.Tensor, h: torch.Tensor, y: torch.Tensor, **norm) -> None:
        """``h += sum_ranks(x_part @ w^T) [* gate]`` and ``y = norm(h)`` over the peer group (one GEMM, one reduce kernel)."""
        self.st.linear_reduce(x_part, w, residual=h, y=y, **norm)

    def images(self) -> None:
        """This rank's cameras through the tower and the projector, then the projected rows of all cameras."""
        v, proj = self.cfg.vision, self.model.vision.projector
        n = self.img_hi - self.img_lo
        self.vision(self.img_lo, self.img_hi)
        if n > 0:
            ops.gemm(self.v_x[: n * v.num_patches], proj.weight, self.v_proj[: n * v.num_patches], bias=proj.bias)
        self.st_img.all_gather_rows(self.v_proj, out=self.v_all)

    def prefix(self, lang_bucket: int, kv_events=None) -> None:
        cfg, t, lm = self.cfg, self.cfg.text, self.model.paligemma_lm
        n_per = self.img_tokens + lang_bucket
        Mp = self.B * n_per
        if self.B == 1 and not self._prefix_splits_env:
            self.prefix_splits = 4 if n_per >= 896 else 2
        h, x = self.p_h[:Mp], self.p_x[:Mp]
        for b in range(self.B):
            h[b * n_per: b * n_per + self.img_tokens].copy_(self.v_all[b * self.img_tokens:(b + 1) * self.img_tokens])
        ops.embedding(self.input_ids.view(-1), lm.embed_tokens, h, scale=lm.embed_scale, dst_rows=self.lang_rows)
        Hq, D = self.Hq, t.head_dim
        qkv, q, attn, act = self.p_qkv[:Mp], self.p_q[:Mp], self.p_attn[:Mp], self.p_act[:Mp]
        q3, a3 = q.unflatten(1, (Hq, D)), attn.unflatten(1, (Hq, D))
        last = len(lm.layers) - 1
        eps = t.rms_norm_eps
        ops.norm(h, "gemma_rms", weight=lm.layers[0].input_layernorm.weight, eps=eps, out=x)
        if self.scatter:
            return self._prefix_scatter(h, x, qkv, q3, attn, a3, act, n_per, kv_events)
        for li, layer in enumerate(lm.layers):
            kpool, vpool = self.pool.layer(li)
            ops.gemm(x, self.tp_pqkv[li], qkv, rope=self.p_rope[li])
            if kv_events is not None:
                kv_events[li].record(torch.cuda.current_stream())     # this block's prefix K / V are in the pool
            if li == last:
                break  # only this block's K/V are consumed downstream
            ops.attention(q3, kpool, vpool, a3, self.p_qstart, self.p_qlen, self.p_kvptr, self.p_kvlen,
                          max_q_len=n_per, splits=self.prefix_splits, sm_scale=D ** -0.5)
            self._reduce(attn, layer.attn.o.weight, h, x, norm="gemma_rms", weight=layer.post_attention_layernorm.weight, eps=eps)
            ops.gemm(x, layer.mlp.gate_up.weight, act, act="gelu_tanh", glu=True)
            self._reduce(act, layer.mlp.down.weight, h, x, norm="gemma_rms", weight=lm.layers[li + 1].input_layernorm.weight, eps=eps)

    def _prefix_scatter(self, h, x, qkv, q3, attn, a3, act, n_per, kv_events=None) -> None:
        """Prefix blocks with a sequence-parallel residual: each product's tiles go to the rank that owns the rows,
        which sums them, adds its residual rows, applies the next norm and stores the normalised rows into every
        rank's gathered matrix; the next GEMM waits for those rows in its loader (all-gather fused into the GEMM)."""
        t, lm, st = self.cfg.text, self.model.paligemma_lm, self.st_sc
        D, eps = t.head_dim, t.rms_norm_eps
        last = len(lm.layers) - 1
        y, wait = x, None
        for li, layer in enumerate(lm.layers):
            kpool, vpool = self.pool.layer(li)
            ops.gemm(y, self.tp_pqkv[li], qkv, rope=self.p_rope[li], wait=wait)
            if kv_events is not None:
                kv_events[li].record(torch.cuda.current_stream())
            if li == last:
                break
            ops.attention(q3, kpool, vpool, a3, self.p_qstart, self.p_qlen, self.p_kvptr, self.p_kvlen,
                          max_q_len=n_per, splits=self.prefix_splits, sm_scale=D ** -0.5)
            t1 = st.linear_reduce(attn, layer.attn.o.weight, scatter=True, residual=h, norm="gemma_rms",
                                  weight=layer.post_attention_layernorm.weight, eps=eps, gather=True)
            ops.gemm(t1.y, layer.mlp.gate_up.weight, act, act="gelu_tanh", glu=True, wait=t1.wait)
            t2 = st.linear_reduce(act, layer.mlp.down.weight, scatter=True, residual=h, norm="gemma_rms",
                                  weight=lm.layers[li + 1].input_layernorm.weight, eps=eps, gather=True)
            y, wait = t2.y, t2.wait

    def expert(self) -> None:
        if self.expert_replicated:
            return PI05Plan.expert(self)
        cfg, e, t = self.cfg, self.cfg.expert, self.cfg.text
        heads, stack = self.model.heads, self.model.expert_stack
        Hq, D, He, Me = self.Hq_e, t.head_dim, e.hidden_size, self.Me
        h, x = self.e_h, self.e_x
        q3, a3 = self.e_q.unflatten(1, (Hq, D)), self.e_attn.unflatten(1, (Hq, D))
        n_layers, eps = len(stack.layers), e.rms_norm_eps
        self.x_t.copy_(self.noise.view(Me, -1))
        for i in range(cfg.num_inference_steps):
            ops.gemm(self.x_t, heads.action_in_proj.weight, h, bias=heads.action_in_proj.bias)
            ops.norm(h, "ada_rms", mod=self.mod_in[0][i:i + 1], group=Me, eps=eps, out=x)
            for li, layer in enumerate(stack.layers):
                kpool, vpool = self.pool.layer(li)
                m_in, m_post = self.mod_in[li][i], self.mod_post[li][i]
                nxt = self.mod_in[li + 1][i] if li + 1 < n_layers else self.mod_final[i]
                ops.gemm(x, self.tp_eqkv[li], self.e_qkv, rope=self.rope_desc[li])
                ops.attention(q3, kpool, vpool, a3, self.e_qstart, self.e_qlen, self.e_kvptr, self.e_kvlen,
                              max_q_len=self.C, splits=self.expert_splits, sm_scale=D ** -0.5)
                self._reduce(self.e_attn, layer.attn.o.weight, h, x, col_gate=m_in[2 * He:], norm="ada_rms", mod=m_post, eps=eps)
                ops.gemm(x, layer.mlp.gate_up.weight, self.e_act, act="gelu_tanh", glu=True)
                self._reduce(self.e_act, layer.mlp.down.weight, h, x, col_gate=m_post[2 * He:], norm="ada_rms", mod=nxt, eps=eps)
            ops.gemm(x, heads.action_out_proj.weight, self.e_v, bias=heads.action_out_proj.bias)
            ops.axpy(self.x_t, self.e_v, self.dt)
        self.out.view(Me, -1).copy_(self.x_t)



__all__ = ["PI05TPPlan", "split_cameras"]
