"""Static execution plan of Pi0 on B200 (vision and prefix stages are Pi0.5's).

Expert stage: one pass for the state token of every robot (its K/V land in the slot right
behind the robot's real prefix rows), then the 10-step Euler loop over the action tokens,
whose K/V follow the state slot, so every attention call reads one contiguous slot range.
The ``cat(action_emb, time_emb) -> Linear(2H, H)`` of the reference is evaluated as
``W_a (W_in x + b_in) + (W_t time_emb + b)``: the two input projections are folded into one
``(H, action_dim)`` weight at set-up and the time half becomes a per-step bias row.
"""

from __future__ import annotations

import torch

from ... import ops
from ..pi05.plan_pi05 import PI05Layout, PI05Plan
from .modeling_pi0 import PI0Model


class PI0Plan(PI05Plan):
    suffix_extra = 1

    def __init__(self, model: PI0Model, *, max_batch_size: int = 1, num_images: int = 3, device="cuda",
                 quantization: str | None = None) -> None:
        # block-scaled fp8 covers the shared prefix decoder; the Pi0 expert keeps its bf16 launch sequence
        super().__init__(model, max_batch_size=max_batch_size, num_images=num_images, device=device, quantization=quantization)
        cfg, dev, B = self.cfg, self.device, self.B
        He = cfg.expert.hidden_size
        bf = torch.bfloat16
        self.state = torch.zeros(B, cfg.max_state_dim, dtype=bf, device=dev)
        self.s_h = torch.zeros(B, He, dtype=bf, device=dev)
        self.s_x = torch.zeros(B, He, dtype=bf, device=dev)
        self.s_qkv = torch.zeros(B, self.e_qkv.shape[1], dtype=bf, device=dev)
        self.s_q = torch.zeros(B, self.e_q.shape[1], dtype=bf, device=dev)
        self.s_attn = torch.zeros(B, self.e_q.shape[1], dtype=bf, device=dev)
        self.s_act = torch.zeros(B, self.I_e, dtype=bf, device=dev)
        self.s_pos = torch.zeros(B, dtype=torch.int32, device=dev)
        self.s_slots = torch.zeros(B, dtype=torch.int64, device=dev)
        self.s_qstart = torch.arange(B, dtype=torch.int32, device=dev)
        self.s_qlen = torch.ones(B, dtype=torch.int32, device=dev)
        self.s_kvlen = torch.zeros(B, dtype=torch.int32, device=dev)
        self.e_t = torch.zeros(self.Me, He, dtype=bf, device=dev)
        self.w_fold: torch.Tensor | None = None
        self.time_bias: torch.Tensor | None = None

    @torch.no_grad()
    def build_modulation_tables(self) -> None:
        """Fold the action/time input projections (call after weights are loaded)."""
        cfg, heads = self.cfg, self.model.heads
        H, N = cfg.expert.hidden_size, cfg.num_inference_steps
        w = heads.action_time_mlp_in.weight.float()
        wa, wt = w[:, :H], w[:, H:]
        self.w_fold = (wa @ heads.action_in_proj.weight.float()).to(torch.bfloat16).contiguous()
        ts = 1.0 + torch.arange(N, dtype=torch.float32, device=self.device) * self.dt
        te = heads.time_embedding(ts).to(torch.bfloat16).float()
        bias = te @ wt.t() + heads.action_time_mlp_in.bias.float() + wa @ heads.action_in_proj.bias.float()
        self.time_bias = bias.to(torch.bfloat16).contiguous()
        if self.fp8:
            self._build_fp8_weights(expert=False)
        if self.fold_norms:
            self._fold_prefix()
            # Gemma RMSNorm weights (1 + w) folded into the weights that consume the normed rows; the
            # per-row 1/rms is applied in that GEMM's epilogue from sums of squares accumulated by the
            # epilogue of the GEMM that wrote the rows (the first block of a pass keeps its norm kernel).
            def fold(w, norm_w):
                return (w.float() * (1.0 + norm_w.float())[None, :]).to(torch.bfloat16).contiguous()

            stack = self.model.expert_stack
            t = cfg.text
            Hq, Hkv, D = self.Hq_e, self.Hkv, t.head_dim
            # QKV rows reordered for the rotating epilogue; block 0 keeps its norm kernel and the plain weight
            self.fold_qkv = [ops.permute_rope_rows(fold(l.attn.qkv.weight, l.input_layernorm.weight) if li > 0
                                                   else l.attn.qkv.weight, Hq, Hkv, D)
                             for li, l in enumerate(stack.layers)]
            self.e_rope = self._rope_descs(self.e_q, self.e_pos, self.e_slots, self.Hq_e)
            self.s_rope = self._rope_descs(self.s_q, self.s_pos, self.s_slots, self.Hq_e)
            self.fold_gate_up = [fold(l.mlp.gate_up.weight, l.post_attention_layernorm.weight) for l in stack.layers]
            self.fold_out = fold(heads.action_out_proj.weight, stack.norm.weight)
            self.e_ss = torch.zeros(2, self.Me, dtype=torch.float32, device=self.device)
            self.s_ss = torch.zeros(2, self.B, dtype=torch.float32, device=self.device)

    def set_layout(self, layout: PI05Layout) -> bool:
        changed = super().set_layout(layout)
        if changed:
            real, base = self._real, self._base
            self.s_pos.copy_(torch.tensor(real, dtype=torch.int32))
            self.s_slots.copy_(torch.tensor([b + r for b, r in zip(base, real)], dtype=torch.int64))
            self.s_kvlen.copy_(torch.tensor([r + 1 for r in real], dtype=torch.int32))
        return changed

    def _block(self, layer, li, h, x, qkv, q, attn, act, pos, slots, qstart, qlen, kvlen, max_q, splits,
               ss=None, rope=None) -> None:
        t, e = self.cfg.text, self.cfg.expert
        Hq, Hkv, D = self.Hq_e, self.Hkv, t.head_dim
        kpool, vpool = self.pool.layer(li)
        if ss is not None:
            rms = (e.hidden_size, e.rms_norm_eps)
            if li == 0:
                ops.norm(h, "gemma_rms", weight=layer.input_layernorm.weight, eps=e.rms_norm_eps, out=x)
                ops.gemm(x, self.fold_qkv[li], qkv, rope=rope[li])
            else:
                ops.gemm(h, self.fold_qkv[li], qkv, row_scale=ss[0], row_rms=rms, rope=rope[li])
            ops.attention(q.unflatten(1, (Hq, D)), kpool, vpool, attn.unflatten(1, (Hq, D)), qstart, qlen,
                          self.e_kvptr, kvlen, max_q_len=max_q, splits=splits, sm_scale=D ** -0.5)
            # each accumulating GEMM clears the other accumulator, which is idle at that point
            ops.gemm(attn, layer.attn.o.weight, h, residual=h, sumsq=ss[1], zero=ss[0])
            ops.gemm(h, self.fold_gate_up[li], act, row_scale=ss[1], row_rms=rms, act="gelu_tanh", glu=True)
            ops.gemm(act, layer.mlp.down.weight, h, residual=h, sumsq=ss[0], zero=ss[1])
            return
        ops.norm(h, "gemma_rms", weight=layer.input_layernorm.weight, eps=e.rms_norm_eps, out=x)
        ops.gemm(x, layer.attn.qkv.weight, qkv)
        ops.rope_kv(qkv, Hq, Hkv, D, q, pos=pos, cos_sin=self.cos_sin, k_pool=kpool, v_pool=vpool, slots=slots)
        ops.attention(q.unflatten(1, (Hq, D)), kpool, vpool, attn.unflatten(1, (Hq, D)), qstart, qlen, self.e_kvptr,
                      kvlen, max_q_len=max_q, splits=splits, sm_scale=D ** -0.5)
        ops.gemm(attn, layer.attn.o.weight, h, residual=h)
        ops.norm(h, "gemma_rms", weight=layer.post_attention_layernorm.weight, eps=e.rms_norm_eps, out=x)
        ops.gemm(x, layer.mlp.gate_up.weight, act, act="gelu_tanh", glu=True)
        ops.gemm(act, layer.mlp.down.weight, h, residual=h)

    def expert(self) -> None:
        self.state_pass()
        self.euler_loop()

    def _first_step_overlappable(self) -> bool:
        return False           # this plan's own run() puts the state-token pass on the second stream

    def state_pass(self, before_block=None) -> None:
        """The state token of every robot through the expert, once per request. ``before_block(li)`` runs before
        block ``li`` is issued (the overlapped schedule waits there for the prefix K/V of that block: the padded
        prompt rows of the prefix land in the pool slot the state token uses, so the wait precedes the block)."""
        heads, stack, fold = self.model.heads, self.model.expert_stack, self.fold_norms
        ops.gemm(self.state, heads.state_proj.weight, self.s_h, bias=heads.state_proj.bias)
        for li, layer in enumerate(stack.layers):
            if before_block is not None:
                before_block(li)
            self._block(layer, li, self.s_h, self.s_x, self.s_qkv, self.s_q, self.s_attn, self.s_act, self.s_pos,
                        self.s_slots, self.s_qstart, self.s_qlen, self.s_kvlen, 1, self.expert_splits,
                        ss=self.s_ss if fold else None, rope=self.s_rope if fold else None)

    def run(self, lang_bucket: int) -> torch.Tensor:
        """As the Pi0.5 plan; with the overlapped schedule the state-token pass (90 small launches) runs on a second
        stream underneath the prefix decoder, block by block behind the prefix K/V it attends to."""
        if not (self.overlap_first_step and self.fold_norms and self.device.type == "cuda"):
            return super().run(lang_bucket)
        main = torch.cuda.current_stream()
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device)
        side = self._side_stream
        fork, join = torch.cuda.Event(), torch.cuda.Event()
        kv_ready = [torch.cuda.Event() for _ in range(self.cfg.num_layers)]
        fork.record(main)
        self.vision()
        self.prefix(lang_bucket, kv_events=kv_ready)
        with torch.cuda.stream(side):
            side.wait_event(fork)
            self.state_pass(before_block=lambda li: side.wait_event(kv_ready[li]))
            join.record(side)
        main.wait_event(join)
        self.euler_loop()
        return self.out

    def euler_loop(self) -> None:
        cfg, heads, stack = self.cfg, self.model.heads, self.model.expert_stack
        Me, fold = self.Me, self.fold_norms
        self.x_t.copy_(self.noise.view(Me, -1))
        for i in range(cfg.num_inference_steps):
            ops.gemm(self.x_t, self.w_fold, self.e_t, bias=self.time_bias[i], act="silu")
            ops.gemm(self.e_t, heads.action_time_mlp_out.weight, self.e_h, bias=heads.action_time_mlp_out.bias)
            for li, layer in enumerate(stack.layers):
                self._block(layer, li, self.e_h, self.e_x, self.e_qkv, self.e_q, self.e_attn, self.e_act, self.e_pos,
                            self.e_slots, self.e_qstart, self.e_qlen, self.e_kvlen, self.C, self.expert_splits,
                            ss=self.e_ss if fold else None, rope=self.e_rope if fold else None)
            if fold:
                ops.gemm(self.e_h, self.fold_out, self.e_v, bias=heads.action_out_proj.bias, row_scale=self.e_ss[0],
                         row_rms=(cfg.expert.hidden_size, cfg.expert.rms_norm_eps))
            else:
                ops.norm(self.e_h, "gemma_rms", weight=stack.norm.weight, eps=cfg.expert.rms_norm_eps, out=self.e_x)
                ops.gemm(self.e_x, heads.action_out_proj.weight, self.e_v, bias=heads.action_out_proj.bias)
            ops.axpy(self.x_t, self.e_v, self.dt)
        self.out.view(Me, -1).copy_(self.x_t)


__all__ = ["PI0Plan"]
