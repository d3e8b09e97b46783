"""The persistent action-expert kernel against a plain PyTorch fp32 statement of the same loop."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _reference(w, tabs, geo, k_pool, v_pool, kv_ptr, kv_len, pos, cos_sin, x0, eps, dt, sm_scale, step_begin, step_end):
    """fp32 restatement: AdaRMS-modulated Gemma blocks attending into [pool rows | own K/V], Euler update."""
    M, H, Hq, D = geo.rows, geo.hidden, geo.q_heads, geo.head_dim
    Lp = kv_len - M
    x = x0.float().clone()
    cs = cos_sin[pos.long()].float()
    cos, sin = cs[:, : D // 2], cs[:, D // 2:]

    def rope(t):                       # (M, heads, D)
        a, b = t[..., : D // 2], t[..., D // 2:]
        return torch.cat([a * cos[:, None] - b * sin[:, None], b * cos[:, None] + a * sin[:, None]], dim=-1)

    def rms(h):
        return h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)

    for i in range(step_begin, step_end):
        h = x.bfloat16().float() @ w["w_in"].float().t() + w["b_in"].float()
        for li in range(geo.layers):
            wq, wo, wgu, wd = (t.float() for t in w["layers"][li])
            xin = (rms(h) * tabs["in_scale"][i, li]).bfloat16().float()       # the kernel rounds h * scale; 1/rms is applied after the product
            qkv = (xin @ wq.t() + tabs["qkv_bias"][i, li]).bfloat16().float()
            q = rope(qkv[:, : Hq * D].reshape(M, Hq, D)).bfloat16().float()
            k = rope(qkv[:, Hq * D:(Hq + 1) * D].reshape(M, 1, D)).bfloat16().float()
            v = qkv[:, (Hq + 1) * D:].reshape(M, 1, D)
            kk = torch.cat([k_pool[li, kv_ptr:kv_ptr + Lp, 0].float(), k[:, 0]])
            vv = torch.cat([v_pool[li, kv_ptr:kv_ptr + Lp, 0].float(), v[:, 0]])
            s = torch.einsum("mhd,kd->mhk", q, kk) * sm_scale
            a = torch.einsum("mhk,kd->mhd", torch.softmax(s, dim=-1), vv).reshape(M, Hq * D).bfloat16().float()
            h = h + tabs["gate_in"][i, li] * (a @ wo.t())
            xin = (rms(h) * tabs["post_scale"][i, li]).bfloat16().float()
            gu = xin @ wgu.t() + tabs["gu_bias"][i, li]
            act = (torch.nn.functional.gelu(gu[:, 0::2], approximate="tanh") * gu[:, 1::2]).bfloat16().float()
            h = h + tabs["gate_post"][i, li] * (act @ wd.t())
        vel = (rms(h) * tabs["fin_scale"][i]) @ w["w_out"].float().t() + tabs["out_bias"][i]
        x = x + dt * vel
    return x


def _case(layers, steps, prefix_rows, M=50, H=1024, I=4096, Hq=8, seed=0, step_begin=0):
    from phyai_b200 import ops
    from phyai_b200.ops.expert_stack import ExpertGeometry, ExpertStack

    D, A = 256, 32
    geo = ExpertGeometry(rows=M, hidden=H, inter=I, q_heads=Hq, head_dim=D, action_dim=A, layers=layers, steps=steps)
    assert ExpertStack.supports(geo, prefix_rows + M)
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0, dtype=torch.bfloat16):
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)

    Nqkv = (Hq + 2) * D
    w = dict(layers=[(rnd(Nqkv, H, std=H ** -0.5), rnd(H, Hq * D, std=(Hq * D) ** -0.5), rnd(2 * I, H, std=H ** -0.5),
                      rnd(H, I, std=I ** -0.5)) for _ in range(layers)],
             w_in=rnd(H, A, std=A ** -0.5), b_in=rnd(H, std=0.1), w_out=rnd(A, H, std=H ** -0.5))
    f32 = torch.float32
    tabs = dict(in_scale=1 + rnd(steps, layers, H, std=0.2, dtype=f32), post_scale=1 + rnd(steps, layers, H, std=0.2, dtype=f32),
                gate_in=rnd(steps, layers, H, std=0.5, dtype=f32), gate_post=rnd(steps, layers, H, std=0.5, dtype=f32),
                qkv_bias=rnd(steps, layers, Nqkv, std=0.2, dtype=f32), gu_bias=rnd(steps, layers, 2 * I, std=0.2, dtype=f32),
                fin_scale=1 + rnd(steps, H, std=0.2, dtype=f32), out_bias=rnd(steps, A, std=0.2, dtype=f32))
    slots = 1 + prefix_rows + M + 3
    k_pool, v_pool = rnd(layers, slots, 1, D), rnd(layers, slots, 1, D)
    kv_ptr = torch.tensor([1], dtype=torch.int32, device=DEV)
    kv_len = torch.tensor([prefix_rows + M], dtype=torch.int32, device=DEV)
    pos = (prefix_rows + torch.arange(M, dtype=torch.int32)).to(DEV)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.arange(prefix_rows + M + 8, dtype=torch.float32)[:, None] * inv
    cos_sin = torch.cat([ang.cos(), ang.sin()], dim=-1).to(DEV).contiguous()
    x0 = rnd(M, A)
    out = torch.zeros(M, A, dtype=torch.bfloat16, device=DEV)
    st = ExpertStack(geo, device=DEV)
    st.set_weights(w["layers"])
    st.set_tables(**tabs)
    eps, dt, sm = 1e-6, -1.0 / steps, D ** -0.5
    kw = dict(w_in=w["w_in"], b_in=w["b_in"], w_out=w["w_out"], k_pool=k_pool, v_pool=v_pool, kv_ptr=kv_ptr, kv_len=kv_len,
              pos=pos, cos_sin=cos_sin, x0=x0, out=out, eps=eps, dt=dt, sm_scale=sm, step_begin=step_begin, step_end=steps)
    st.run(**kw)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    ref = _reference(w, tabs, geo, k_pool, v_pool, 1, prefix_rows + M, pos, cos_sin, x0, eps, dt, sm, step_begin, steps)
    torch.testing.assert_close(out.float(), ref, atol=5e-2, rtol=5e-2)
    # a second launch on the same object starts from clean scratch
    out2 = torch.zeros_like(out)
    kw["out"] = out2
    st.run(**kw)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    torch.testing.assert_close(out2.float(), ref, atol=5e-2, rtol=5e-2)
    return st


def test_expert_stack_full_width_short_prefix():
    _case(layers=2, steps=2, prefix_rows=200)


def test_expert_stack_full_width_long_prefix_and_step_offset():
    # 968 + 50 rows: every attention unit holds a full 64-key tile except the last; starts at the second step
    _case(layers=2, steps=3, prefix_rows=968, seed=1, step_begin=1)


def test_expert_stack_narrow_geometry_with_idle_ctas():
    # 40 / 32 / 8 / 4 (tile, K block) pairs per projection: most CTAs own no pair in a phase
    _case(layers=3, steps=2, prefix_rows=77, M=50, H=128, I=256, Hq=8, seed=2)


def test_expert_stack_inside_graph():
    from phyai_b200 import ops

    st = _case(layers=1, steps=1, prefix_rows=130, seed=3)
    del st
    # capture + replay twice with new inputs
    from phyai_b200.ops.expert_stack import ExpertGeometry, ExpertStack

    geo = ExpertGeometry(rows=50, hidden=1024, inter=4096, q_heads=8, head_dim=256, action_dim=32, layers=1, steps=2)
    g = torch.Generator().manual_seed(5)

    def rnd(*shape, std=1.0, dtype=torch.bfloat16):
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)

    H, I, Hq, D, A, M, P = 1024, 4096, 8, 256, 32, 50, 300
    w = dict(layers=[(rnd(10 * D, H, std=H ** -0.5), rnd(H, 8 * D, std=(8 * D) ** -0.5), rnd(2 * I, H, std=H ** -0.5), rnd(H, I, std=I ** -0.5))],
             w_in=rnd(H, A, std=A ** -0.5), b_in=rnd(H, std=0.1), w_out=rnd(A, H, std=H ** -0.5))
    f32 = torch.float32
    tabs = dict(in_scale=1 + rnd(2, 1, H, std=0.2, dtype=f32), post_scale=1 + rnd(2, 1, H, std=0.2, dtype=f32),
                gate_in=rnd(2, 1, H, std=0.5, dtype=f32), gate_post=rnd(2, 1, H, std=0.5, dtype=f32),
                qkv_bias=rnd(2, 1, 10 * D, std=0.2, dtype=f32), gu_bias=rnd(2, 1, 2 * I, std=0.2, dtype=f32),
                fin_scale=1 + rnd(2, H, std=0.2, dtype=f32), out_bias=rnd(2, A, std=0.2, dtype=f32))
    k_pool, v_pool = rnd(1, P + M + 4, 1, D), rnd(1, P + M + 4, 1, D)
    kv_ptr = torch.tensor([1], dtype=torch.int32, device=DEV)
    kv_len = torch.tensor([P + M], dtype=torch.int32, device=DEV)
    pos = (P + torch.arange(M, dtype=torch.int32)).to(DEV)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.arange(P + M + 8, dtype=torch.float32)[:, None] * inv
    cos_sin = torch.cat([ang.cos(), ang.sin()], dim=-1).to(DEV).contiguous()
    x0, out = rnd(M, A), torch.zeros(M, A, dtype=torch.bfloat16, device=DEV)
    st = ExpertStack(geo, device=DEV)
    st.set_weights(w["layers"])
    st.set_tables(**tabs)
    kw = dict(w_in=w["w_in"], b_in=w["b_in"], w_out=w["w_out"], k_pool=k_pool, v_pool=v_pool, kv_ptr=kv_ptr, kv_len=kv_len,
              pos=pos, cos_sin=cos_sin, x0=x0, out=out, eps=1e-6, dt=-0.5, sm_scale=D ** -0.5)
    st.run(**kw)                        # first call outside capture (sets the kernel's attributes)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        st.run(**kw)
    for seed in (7, 8):
        x0.copy_(torch.randn(M, A, generator=torch.Generator().manual_seed(seed)).to(DEV))
        graph.replay()
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0
        ref = _reference(w, tabs, geo, k_pool, v_pool, 1, P + M, pos, cos_sin, x0, 1e-6, -0.5, D ** -0.5, 0, 2)
        torch.testing.assert_close(out.float(), ref, atol=5e-2, rtol=5e-2)
