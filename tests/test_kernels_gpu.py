"""Numerics of the sm_100a kernels against plain PyTorch fp32 restatements of the same ops."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 2e-2  # bf16 outputs


def relerr(a, b):
    a, b = a.float(), b.float()
    return float((a - b).abs().max() / (b.abs().max() + 1e-6))


def _status_ok():
    from phyai_b200 import ops

    torch.cuda.synchronize()
    assert ops.kernel_status() == 0


GEMM_CASES = [
    dict(M=128, N=128, K=64, force_swap=0, force_bn=128, force_splits=1),
    dict(M=256, N=256, K=512, force_swap=0),
    dict(M=968, N=2560, K=2048),
    dict(M=968, N=4096, K=2048, glu=True, act="gelu_tanh"),
    dict(M=968, N=2048, K=2048, residual=True, force_bn=128),
    dict(M=768, N=4304, K=1152, bias=True, act="gelu_tanh"),
    dict(M=768, N=1152, K=4304, bias=True, residual=True),
    dict(M=768, N=1152, K=592, bias=True, residual=True, res_mod=256),
    dict(M=50, N=2560, K=1024),
    dict(M=50, N=1024, K=2048, residual=True, col_gate=True),
    dict(M=50, N=8192, K=1024, glu=True, act="gelu_tanh"),
    dict(M=50, N=1024, K=4096, residual=True, col_gate=True, force_splits=4),
    dict(M=50, N=32, K=1024, bias=True),
    dict(M=50, N=1024, K=32, bias=True),
    dict(M=1, N=1024, K=1024, bias=True, act="silu"),
    dict(M=200, N=1024, K=1024, row_scale=True),
    dict(M=400, N=2048, K=1024, glu=True, act="silu"),
    dict(M=300, N=512, K=1024, force_swap=0, force_bn=64),
    dict(M=300, N=512, K=1024, force_swap=0, force_bn=32, out_fp32=True),
    dict(M=768, N=3456, K=1152, bias=True),                                           # picks the 192-wide tile
    dict(M=700, N=1000, K=320, force_swap=0, force_bn=192, bias=True, residual=True),  # 192-wide, ragged N and M edges
    dict(M=640, N=1536, K=512, force_swap=0, force_bn=192, glu=True, act="silu", force_splits=2),
]


@pytest.mark.parametrize("case", GEMM_CASES, ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
def test_gemm(case):
    from phyai_b200 import ops
    from phyai_b200.ops import ref

    c = dict(case)
    M, N, K = c.pop("M"), c.pop("N"), c.pop("K")
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    glu, act = c.pop("glu", False), c.pop("act", "none")
    No = N // 2 if glu else N
    kw = {}
    if c.pop("bias", False):
        kw["bias"] = torch.randn(N, device=DEV, generator=g).bfloat16()
    res_mod = c.pop("res_mod", 0)
    if c.pop("residual", False):
        kw["residual"] = torch.randn(res_mod or M, No, device=DEV, generator=g).bfloat16()
        kw["res_mod"] = res_mod
    if c.pop("col_gate", False):
        kw["col_gate"] = torch.randn(No, device=DEV, generator=g).bfloat16()
    if c.pop("row_scale", False):
        kw["row_scale"] = torch.rand(M, device=DEV, generator=g) + 0.5
    odt = torch.float32 if c.pop("out_fp32", False) else torch.bfloat16
    out = ops.gemm(x, w, act=act, glu=glu, out_dtype=odt, **kw, **c)
    _status_ok()
    exp = ref.gemm(x, w, act=act, glu=glu, out_dtype=odt, **kw)
    assert relerr(out, exp) < TOL


def test_gemm_sumsq_and_determinism():
    from phyai_b200 import ops

    for M in (50, 968):
        x = (torch.randn(M, 2048, device=DEV) * 0.5).bfloat16()
        w = (torch.randn(1024, 2048, device=DEV) * 0.05).bfloat16()
        ss = torch.zeros(M, device=DEV)
        o = ops.gemm(x, w, sumsq=ss)
        o2 = ops.gemm(x, w)
        _status_ok()
        assert relerr(ss, o.float().pow(2).sum(-1)) < 1e-4
        assert torch.equal(o, o2)
        if M > 256:      # 192-wide tiles: the last column block of a tile is only half populated
            ss3 = torch.zeros(M, device=DEV)
            o3 = ops.gemm(x, w, sumsq=ss3, force_swap=0, force_bn=192)
            _status_ok()
            assert relerr(ss3, o3.float().pow(2).sum(-1)) < 1e-4 and relerr(o3, o) < 1e-2


@pytest.mark.parametrize("M,glu", [(50, False), (50, True), (1, False), (300, True)])
def test_gemm_folded_rms_norm(M, glu):
    """norm(h) @ W^T as one GEMM: (1 + scale) folded into W, shift @ W^T as a bias, 1/rms in the epilogue."""
    from phyai_b200 import ops

    K, N, eps = 1024, 2048, 1e-6
    g = torch.Generator(device="cpu").manual_seed(M)
    h0 = (torch.randn(M, K, generator=g) * 2).bfloat16().to(DEV)
    wo = (torch.randn(K, K, generator=g) * 0.03).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    scale, shift = (torch.randn(K, generator=g) * 0.3).to(DEV), (torch.randn(K, generator=g) * 0.3).to(DEV)
    ss = torch.full((2, M), 7.0, device=DEV)                       # dirty: the rope launch clears it
    qkv, q = torch.zeros(M, 3 * 64, device=DEV).bfloat16(), torch.zeros(M, 64, device=DEV).bfloat16()
    ops.rope_kv(qkv, 1, 1, 64, q, zero=ss)
    assert float(ss.abs().max()) == 0.0
    h = ops.gemm(h0, wo, residual=h0, sumsq=ss[1])                 # producer: h and its row sums of squares
    w_fold = (w.float() * (1 + scale)[None, :]).bfloat16()
    bias = (shift @ w.float().T).bfloat16()
    act = "gelu_tanh" if glu else "none"
    out = ops.gemm(h, w_fold, bias=bias, row_scale=ss[1], row_rms=(K, eps), act=act, glu=glu)
    _status_ok()
    hf = h.float()
    x = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * (1 + scale) + shift
    y = x @ w.float().T
    if glu:
        y = torch.nn.functional.gelu(y[:, 0::2], approximate="tanh") * y[:, 1::2]
    assert relerr(out, y) < 2e-2, relerr(out, y)


@pytest.mark.parametrize("M,N,K,act,glu,res", [(7040, 5120, 5120, "none", False, True), (1300, 4096, 1024, "silu", True, False),
                                               (2048, 2560, 320, "gelu_tanh", False, False)])
def test_gemm_cta_pair(M, N, K, act, glu, res):
    """The cta_group::2 kernel (256 x 256 tiles on CTA pairs) against the fp32 reference and the default kernel."""
    from phyai_b200 import ops

    g = torch.Generator(device="cpu").manual_seed(N)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).bfloat16().to(DEV)
    r = torch.randn(M, N // 2 if glu else N, generator=g).bfloat16().to(DEV) if res else None
    base = ops.gemm(x, w, bias=bias, residual=r, act=act, glu=glu)
    n0 = ops.gemm_2cta_launches()
    ops.set_gemm_2cta(True)
    try:
        out = ops.gemm(x, w, bias=bias, residual=r, act=act, glu=glu)
        torch.cuda.synchronize()
    finally:
        ops.set_gemm_2cta(None)
    _status_ok()
    assert ops.gemm_2cta_launches() == n0 + 1
    y = x.float() @ w.float().T + bias.float()
    if glu:
        f = torch.nn.functional.silu if act == "silu" else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
        y = f(y[:, 0::2]) * y[:, 1::2]
    elif act == "gelu_tanh":
        y = torch.nn.functional.gelu(y, approximate="tanh")
    if res:
        y = y + r.float()
    assert relerr(out, y) < 2e-2, relerr(out, y)
    assert relerr(out, base) < 1e-2


@pytest.mark.parametrize("pair", [False, True])
def test_gemm_persistent_rms_and_sumsq(pair):
    """Row-RMS factor, sum of squares and scratch clearing in the persistent kernels (one CTA per SM / CTA pairs)."""
    from phyai_b200 import ops

    M, K, N, eps = 1300, 1024, 4096, 1e-6
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).bfloat16().to(DEV)
    r = torch.randn(M, N, generator=g).bfloat16().to(DEV)
    ss_in = x.float().pow(2).sum(-1)
    ss_out = torch.zeros(M, device=DEV)
    scratch = torch.full((M,), 2.0, device=DEV)
    n0 = ops.gemm_2cta_launches()
    ops.set_gemm_2cta(pair)
    try:
        out = ops.gemm(x, w, bias=bias, residual=r, row_scale=ss_in, row_rms=(K, eps), sumsq=ss_out, zero=scratch)
        torch.cuda.synchronize()
    finally:
        ops.set_gemm_2cta(None)
    _status_ok()
    assert ops.gemm_2cta_launches() == n0 + int(pair)
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)) @ w.float().T + bias.float() + r.float()
    assert relerr(out, y) < 2e-2, relerr(out, y)
    assert relerr(ss_out, out.float().pow(2).sum(-1)) < 1e-4
    assert float(scratch.abs().max()) == 0.0


def test_gemm_rejects_misaligned():
    from phyai_b200 import ops

    x = torch.randn(16, 68, device=DEV).bfloat16()   # row stride 136 B: not a multiple of 16
    w = torch.randn(64, 68, device=DEV).bfloat16()
    with pytest.raises(RuntimeError):
        ops.gemm(x, w)
    torch.cuda.synchronize()


@pytest.mark.parametrize("M", [200, 968])
def test_gemm_fp8_rowwise(M):
    from phyai_b200 import ops
    from phyai_b200.ops import ref

    x = torch.randn(M, 2048, device=DEV).bfloat16()
    w = (torch.randn(1024, 2048, device=DEV) * 0.05).bfloat16()
    x8, xs = ops.quant_fp8(x)
    w8, ws = ops.quant_fp8(w)
    o = ops.gemm(x8, w8, a_scale=xs, w_scale=ws)
    _status_ok()
    assert relerr(o, ref.gemm(x8.float(), w8.float(), a_scale=xs, w_scale=ws)) < TOL
    assert relerr(o, ref.gemm(x, w)) < 8e-2     # quantisation error itself


ATTN_CASES = [
    dict(B=3, ql=256, kl=256, Hq=16, Hkv=16, D=72),
    dict(B=1, ql=968, kl=968, Hq=8, Hkv=1, D=256, paged=True),
    dict(B=1, ql=50, kl=1018, Hq=8, Hkv=1, D=256, paged=True, splits=8),
    dict(B=2, ql=50, kl=834, Hq=8, Hkv=1, D=256, paged=True, splits=2),
    dict(B=2, ql=100, kl=100, Hq=8, Hkv=2, D=128, causal=True),
    dict(B=1, ql=333, kl=500, Hq=4, Hkv=4, D=128, causal=True, splits=2),
    dict(B=1, ql=10, kl=26, Hq=4, Hkv=1, D=32, paged=True),
    dict(B=2, ql=64, kl=0, Hq=2, Hkv=2, D=64),
    dict(B=1, ql=300, kl=1500, Hq=4, Hkv=2, D=128),
    dict(B=1, ql=700, kl=700, Hq=2, Hkv=1, D=256, causal=True),
    dict(B=2, ql=200, kl=900, Hq=8, Hkv=8, D=64, splits=4),
]


@pytest.mark.parametrize("impl", ["tc", "mma"])
@pytest.mark.parametrize("case", ATTN_CASES, ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
def test_attention(case, impl):
    from phyai_b200 import ops
    from phyai_b200.ops import ref

    B, ql, kl, Hq, Hkv, D = (case[k] for k in ("B", "ql", "kl", "Hq", "Hkv", "D"))
    causal, paged, splits = case.get("causal", False), case.get("paged", False), case.get("splits", 1)
    q = torch.randn(B * ql, Hq, D, device=DEV).bfloat16()
    R = B * kl + 7
    k = torch.randn(R, Hkv, D, device=DEV).bfloat16()
    v = torch.randn(R, Hkv, D, device=DEV).bfloat16()
    ar = torch.arange(B, device=DEV, dtype=torch.int32)
    q_start, q_len = ar * ql, torch.full((B,), ql, device=DEV, dtype=torch.int32)
    kv_ptr, kv_len = ar * kl, torch.full((B,), kl, device=DEV, dtype=torch.int32)
    idx = torch.randperm(R, device=DEV)[: B * kl].int() if paged else None
    o = ops.attention(q, k, v, None, q_start, q_len, kv_ptr, kv_len, kv_indices=idx, max_q_len=ql, causal=causal,
                      splits=splits, impl=impl)
    _status_ok()
    e = ref.attention(q, k, v, q_start.cpu(), q_len.cpu(), kv_ptr.cpu(), kv_len.cpu(), kv_indices=idx, causal=causal)
    assert relerr(o, e) < TOL if kl else float(o.abs().max()) == 0.0


PP_CASES = [
    dict(B=1, ql=256, kl=256, Hq=2, Hkv=2, D=128),
    dict(B=1, ql=700, kl=1000, Hq=5, Hkv=1, D=128),
    dict(B=2, ql=300, kl=515, Hq=4, Hkv=2, D=64),
    dict(B=1, ql=640, kl=640, Hq=2, Hkv=1, D=128, causal=True),
    dict(B=2, ql=130, kl=900, Hq=2, Hkv=2, D=72, causal=True),
    dict(B=1, ql=1500, kl=2100, Hq=3, Hkv=1, D=128, big=True),
]


@pytest.mark.parametrize("case", PP_CASES, ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
def test_attention_pipelined(case):
    """Two-tile ping-pong kernel (P in tensor memory, lazy max) against the fp32 reference."""
    from phyai_b200 import ops
    from phyai_b200.ops import ref

    B, ql, kl, Hq, Hkv, D = (case[k] for k in ("B", "ql", "kl", "Hq", "Hkv", "D"))
    causal = case.get("causal", False)
    scale = 3.0 if case.get("big") else 1.0     # large logits move the running maximum a lot
    q = (torch.randn(B * ql, Hq, D, device=DEV) * scale).bfloat16()
    R = B * kl + 5
    k = torch.randn(R, Hkv, D, device=DEV).bfloat16()
    v = torch.randn(R, Hkv, D, device=DEV).bfloat16()
    ar = torch.arange(B, device=DEV, dtype=torch.int32)
    q_start, q_len = ar * ql, torch.full((B,), ql, device=DEV, dtype=torch.int32)
    kv_ptr, kv_len = ar * kl, torch.full((B,), kl, device=DEV, dtype=torch.int32)
    o = ops.attention(q, k, v, None, q_start, q_len, kv_ptr, kv_len, max_q_len=ql, causal=causal, impl="pp")
    o2 = ops.attention(q, k, v, None, q_start, q_len, kv_ptr, kv_len, max_q_len=ql, causal=causal, impl="pp")
    _status_ok()
    e = ref.attention(q, k, v, q_start.cpu(), q_len.cpu(), kv_ptr.cpu(), kv_len.cpu(), causal=causal)
    assert relerr(o, e) < TOL
    assert torch.equal(o, o2)


@pytest.mark.parametrize("rows,D", [(50, 1024), (968, 2048), (768, 1152), (7, 4096), (3, 12288)])
def test_norms(rows, D):
    from phyai_b200 import ops
    from phyai_b200.ops import ref

    x = torch.randn(rows, D, device=DEV).bfloat16()
    w = (torch.randn(D, device=DEV) * 0.1).bfloat16()
    b = (torch.randn(D, device=DEV) * 0.1).bfloat16()
    assert relerr(ops.norm(x, "rms", weight=w), ref.rms_norm(x, w)) < TOL
    assert relerr(ops.norm(x, "gemma_rms", weight=w), ref.rms_norm(x, w, gemma=True)) < TOL
    assert relerr(ops.norm(x, "layer", weight=w, bias=b), ref.layer_norm(x, w, b)) < TOL
    mod = (torch.randn(1, 3 * D, device=DEV) * 0.2).bfloat16()
    assert relerr(ops.norm(x, "ada_rms", mod=mod, group=rows), ref.ada_rms_norm(x, mod)[0]) < TOL
    modr = (torch.randn(rows, 3 * D, device=DEV) * 0.2).bfloat16()
    assert relerr(ops.norm(x, "ada_rms", mod=modr, group=1), ref.ada_rms_norm(x, modr)[0]) < TOL
    r = torch.randn(rows, D, device=DEV).bfloat16()
    r2 = r.clone()
    y = ops.norm(x, "gemma_rms", weight=w, residual=r2)
    h = (x.float() + r.float()).bfloat16()
    assert relerr(r2, h) < 1e-2 and relerr(y, ref.rms_norm(h, w, gemma=True)) < TOL
    _status_ok()


def test_norm_fp8_outputs():
    from phyai_b200 import ops
    from phyai_b200.ops import ref

    x = torch.randn(64, 1024, device=DEV).bfloat16()
    w = torch.ones(1024, device=DEV).bfloat16()
    for blk in (0, 128):
        y8 = torch.empty(64, 1024, device=DEV, dtype=torch.float8_e4m3fn)
        sc = torch.empty((64, 8) if blk else (64,), device=DEV)
        y = ops.norm(x, "rms", weight=w, y8=y8, y8_scale=sc, y8_block=blk)
        q, s = ref.quant_fp8(y, blk)
        assert relerr(sc, s) < 1e-5 and relerr(y8.float(), q.float()) < 0.08


@pytest.mark.parametrize("M,K", [(50, 1024), (1, 1024), (968, 2048)])
def test_gemm_rope_epilogue(M, K):
    """QKV projection whose epilogue rotates q / k and scatters k / v == GEMM followed by the rope kernel."""
    from phyai_b200 import ops
    from phyai_b200.ops import ref

    Hq, Hkv, D = 8, 1, 256
    N = (Hq + 2 * Hkv) * D
    g = torch.Generator(device="cpu").manual_seed(M + K)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    bias = (torch.randn(N, generator=g) * 0.5).bfloat16().to(DEV)
    pos = (torch.arange(M, dtype=torch.int32) + 3).to(DEV)
    table = ref.rope_cos_sin(torch.arange(0, M + 8, device=DEV), D)
    slots = (torch.randperm(M + 20, generator=g)[:M]).long().to(DEV)
    ss = (torch.rand(M, generator=g) * K * 2 + 1).to(DEV)
    eps = 1e-6

    def pools():
        return torch.zeros(M + 20, Hkv, D, device=DEV, dtype=torch.bfloat16), torch.zeros(M + 20, Hkv, D, device=DEV, dtype=torch.bfloat16)

    # two launches: projection (row-RMS factor and bias in its epilogue), then rotate + scatter
    kp0, vp0 = pools()
    q0 = torch.zeros(M, Hq * D, device=DEV, dtype=torch.bfloat16)
    qkv = ops.gemm(x, w, bias=bias, row_scale=ss, row_rms=(K, eps))
    ops.rope_kv(qkv, Hq, Hkv, D, q0, pos=pos, cos_sin=table, k_pool=kp0, v_pool=vp0, slots=slots)
    # one launch
    kp1, vp1 = pools()
    q1 = torch.zeros_like(q0)
    scratch = torch.full((2, M), 3.0, device=DEV)
    desc = ops.rope_epilogue_desc(q1, kp1, vp1, table, pos, slots, Hq, Hkv, D)
    dummy = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm(x, ops.permute_rope_rows(w, Hq, Hkv, D), dummy, bias=ops.permute_rope_rows(bias, Hq, Hkv, D),
             row_scale=ss, row_rms=(K, eps), rope=desc, zero=scratch)
    _status_ok()
    assert float(scratch.abs().max()) == 0.0 and float(dummy.abs().max()) == 0.0
    assert relerr(q1, q0) < 1e-2, relerr(q1, q0)
    assert relerr(kp1, kp0) < 1e-2 and torch.equal(vp1, vp0)


def test_rope_kv_and_small_ops():
    from phyai_b200 import ops
    from phyai_b200.ops import ref

    M, Hq, Hkv, D = 60, 8, 1, 256
    qkv = torch.randn(M, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    pos = torch.arange(5, 5 + M, device=DEV, dtype=torch.int32)
    table = ref.rope_cos_sin(torch.arange(0, 128, device=DEV), D)
    kp = torch.zeros(100, Hkv, D, device=DEV, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    slots = torch.randperm(100, device=DEV)[:M].long()
    qo = torch.empty(M, Hq * D, device=DEV, dtype=torch.bfloat16)
    ops.rope_kv(qkv, Hq, Hkv, D, qo, pos=pos, cos_sin=table, k_pool=kp, v_pool=vp, slots=slots)
    q3 = qkv[:, : Hq * D].reshape(M, Hq, D)
    k3 = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(M, Hkv, D)
    v3 = qkv[:, (Hq + Hkv) * D:].reshape(M, Hkv, D)
    cs = table[pos.long()]
    assert relerr(qo.reshape(M, Hq, D), ref.apply_rope(q3, cs)) < 1e-2
    assert relerr(kp[slots], ref.apply_rope(k3, cs)) < 1e-2 and torch.equal(vp[slots], v3)
    # per-head RMSNorm before the rotation (Cosmos3 qk-norm)
    nw = (torch.rand(D, device=DEV) + 0.5).bfloat16()
    ops.rope_kv(qkv, Hq, Hkv, D, qo, pos=pos, cos_sin=table, q_norm_w=nw, k_norm_w=nw, k_pool=kp, v_pool=vp, slots=slots)
    assert relerr(qo.reshape(M, Hq, D), ref.apply_rope(ref.rms_norm(q3, nw), cs)) < TOL

    ids = torch.randint(0, 1000, (37,), device=DEV)
    tab = torch.randn(600, 256, device=DEV).bfloat16()
    o = torch.zeros(37, 256, device=DEV, dtype=torch.bfloat16)
    ops.embedding(ids, tab, o, lo=100, hi=700, scale=3.0)
    assert relerr(o, ref.embedding(ids, tab, 100, 700, 3.0)) < 1e-2
    pix = torch.rand(3, 3, 224, 224, device=DEV).bfloat16()
    oc = torch.empty(768, 592, device=DEV, dtype=torch.bfloat16)
    ops.im2col(pix, 14, oc)
    assert torch.equal(oc, ref.im2col(pix, 14, 592))
    x = torch.randn(33, 512, device=DEV).bfloat16()
    for inter in (False, True):
        assert relerr(ops.gated_act(x, "silu", interleaved=inter), ref.gated_act(x, "silu", inter)) < TOL
    c, u = torch.randn(1000, device=DEV).bfloat16(), torch.randn(1000, device=DEV).bfloat16()
    assert relerr(ops.cfg_combine(c, u, 7.0), ref.cfg_combine(c, u, 7.0)) < TOL
    xs = torch.randn(1000, device=DEV)
    xe = xs + (-0.1) * ref.cfg_combine(c, u, 3.0).float()
    ops.cfg_combine(c, u, 3.0, x_fp32=xs, dt=-0.1)
    assert relerr(xs, xe) < 1e-2
    xb = torch.randn(640, device=DEV).bfloat16()
    vb = torch.randn(640, device=DEV).bfloat16()
    e = (xb.float() + 0.25 * vb.float())
    ops.axpy(xb, vb, 0.25)
    assert relerr(xb, e) < 1e-2
    for blk in (0, 128):
        xq = torch.randn(64, 1024, device=DEV).bfloat16()
        y, sc = ops.quant_fp8(xq, blk)
        ye, se = ref.quant_fp8(xq, blk)
        assert relerr(sc, se) < 1e-5 and relerr(y.float(), ye.float()) < 0.08
    _status_ok()


@pytest.mark.parametrize("M,N,K,bias", [(300, 512, 1024, True), (50, 1024, 2048, False), (7, 256, 512, True), (968, 2048, 2048, False),
                                       (129, 392, 384, True)])
def test_gemm_fp8_block_scaled(M, N, K, bias):
    """128x128 weight blocks, 1x128 activation blocks, against the dequantise-then-multiply fp32 restatement."""
    from phyai_b200 import ops
    from phyai_b200.ops import fp8_block

    x = (torch.randn(M, K, device=DEV) * torch.logspace(-1, 1, K // 128, device=DEV).repeat_interleave(128)).bfloat16()
    w = torch.randn(N, K, device=DEV) * 0.05 * torch.logspace(-1, 1, -(-N // 128), device=DEV).repeat_interleave(128)[:N, None]
    b = torch.randn(N, device=DEV).bfloat16() if bias else None
    w8, ws = fp8_block.quantize_weight_block(w)
    x8, xs = ops.quant_fp8(x, 128)
    y = fp8_block.gemm_fp8_block(x8, xs, w8, ws, bias=b)
    _status_ok()
    e = fp8_block.ref_gemm_fp8_block(x8, xs, w8, ws, bias=b)
    assert relerr(y, e) < TOL
    full = x.float() @ w.t() + (b.float() if bias else 0)
    assert relerr(y, full) < 0.08          # quantisation error itself


@pytest.mark.parametrize("rows,D", [(1024, 1024), (7040, 5120), (3001, 2048), (2050, 4096), (1500, 8192), (4099, 2048),
                                    (4100, 4096), (9001, 1024)])
def test_norms_many_rows(rows, D):
    """Row counts that take the warp-per-row kernel."""
    from phyai_b200 import ops
    from phyai_b200.ops import ref

    x = torch.randn(rows, D, device=DEV).bfloat16()
    w = (torch.randn(D, device=DEV) * 0.1).bfloat16()
    assert relerr(ops.norm(x, "rms", weight=w), ref.rms_norm(x, w)) < TOL
    assert relerr(ops.norm(x, "gemma_rms", weight=w), ref.rms_norm(x, w, gemma=True)) < TOL
    modr = (torch.randn(rows // 7 + 1, 3 * D, device=DEV) * 0.2).bfloat16()
    assert relerr(ops.norm(x, "ada_rms", mod=modr, group=7), ref.ada_rms_norm(x, modr.repeat_interleave(7, 0)[:rows])[0]) < TOL
    wide = torch.randn(rows, D + 64, device=DEV).bfloat16()          # rows that are not back to back in memory
    assert relerr(ops.norm(wide[:, :D], "rms", weight=w), ref.rms_norm(wide[:, :D], w)) < TOL
    r = torch.randn(rows, D, device=DEV).bfloat16()
    r2 = r.clone()
    y = ops.norm(x, "rms", weight=w, residual=r2)
    h = (x.float() + r.float()).bfloat16()
    assert relerr(r2, h) < 1e-2 and relerr(y, ref.rms_norm(h, w)) < TOL
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gdn_decode_kernel_matches_the_recurrence(dtype):
    from phyai_b200 import ops
    from phyai_b200.layers.attention.gdn import GatedDeltaNetAttention, gated_delta_rule_recurrent

    g0 = torch.Generator().manual_seed(5)
    B, H, Dk, Dv, steps = 3, 4, 128, 128, 3
    pool = (torch.randn(6, H, Dk, Dv, generator=g0) * 0.2).to(DEV)
    idx = torch.tensor([5, 0, 2], device=DEV)
    ref_state = pool[idx].clone()
    layer = GatedDeltaNetAttention(H, Dk, Dv)
    for _ in range(steps):                       # the pool rows are updated in place, step after step
        q, k = (torch.randn(B, H, Dk, generator=g0).to(DEV, dtype) for _ in range(2))
        v = torch.randn(B, H, Dv, generator=g0).to(DEV, dtype)
        g = (-torch.rand(B, H, generator=g0)).to(DEV, dtype)
        beta = torch.rand(B, H, generator=g0).to(DEV, dtype)
        o = layer.decode(q, k, v, g, beta, state_pool=pool, state_indices=idx)
        o_ref, ref_state = gated_delta_rule_recurrent(q[:, None].float(), k[:, None].float(), v[:, None].float(), g[:, None].float(),
                                                      beta[:, None].float(), ref_state)
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
        torch.testing.assert_close(o.float(), o_ref[:, 0], atol=tol, rtol=tol)
        torch.testing.assert_close(pool[idx], ref_state, atol=1e-4, rtol=1e-4)
    untouched = [i for i in range(6) if i not in (5, 0, 2)]
    assert ops.launch_counter() > 0 and torch.isfinite(pool[untouched]).all()
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_snake_kernel(dtype):
    from phyai_b200.layers.activation import Snake1d

    g0 = torch.Generator().manual_seed(3)
    layer = Snake1d(96, dtype=torch.float32, device=DEV)
    with torch.no_grad():
        layer.alpha.copy_(torch.randn(1, 96, 1, generator=g0) * 0.3)
        layer.beta.copy_(torch.randn(1, 96, 1, generator=g0) * 0.3)
    layer.post_load()
    x = torch.randn(2, 96, 1001, generator=g0).to(DEV, dtype)
    y = layer(x)
    a, b = layer.alpha.float(), layer.beta.float()
    want = x.float() + torch.sin(a * x.float()).pow(2) / (b + 1e-9)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    torch.testing.assert_close(y.float(), want, atol=tol, rtol=tol)
    assert y.dtype == dtype
    _status_ok()


@pytest.mark.parametrize("guided,with_keep", [(False, False), (True, True)])
def test_unipc_step_kernel_matches_fp32_sampler(guided, with_keep):
    """The fused sampler kernel over six steps against the tensor-op sampler run in fp32 on the same velocities."""
    from phyai_b200.models.cosmos3.sampler_unipc import FusedUniPCStream, UniPCMultistepSampler

    g = torch.Generator().manual_seed(3)
    B, C, T, H, W = 2, 4, 5, 6, 8
    n_steps, scale = 6, 3.0
    x0 = torch.randn(B, C, T, H, W, generator=g).bfloat16()
    cond = torch.randn(B, C, T, H, W, generator=g).bfloat16()
    keep = torch.zeros(B, T, dtype=torch.bool)
    keep[:, 0] = keep[1, 3] = True
    vc = [torch.randn(B, C, T, H, W, generator=g).bfloat16() for _ in range(n_steps)]
    vu = [torch.randn(B, C, T, H, W, generator=g).bfloat16() for _ in range(n_steps)]

    ref = UniPCMultistepSampler()
    ref.set_timesteps(n_steps)
    x = x0.float().clone()
    if with_keep:
        x[keep[:, None, :].expand(B, C, T)] = cond.float()[keep[:, None, :].expand(B, C, T)]
    start = x.clone()
    for i in range(n_steps):
        v = vu[i].float() + scale * (vc[i].float() - vu[i].float()) if guided else vc[i].float()
        x = ref.step(v, None, x)
        x = x.bfloat16().float()                    # the sample the model would see is bf16
        if with_keep:
            m = keep[:, None, :].expand(B, C, T)
            x[m] = cond.float()[m]

    fused = UniPCMultistepSampler()
    fused.set_timesteps(n_steps)
    xs = start.bfloat16().cuda().contiguous()
    st = FusedUniPCStream(fused, xs, view=(C, T, H * W), keep=keep.cuda() if with_keep else None, cond=cond.cuda() if with_keep else None)
    for i in range(n_steps):
        if guided:
            st.step(vc[i].cuda(), uncond=vu[i].cuda(), g=scale)
        else:
            st.step(vc[i].cuda())
    _status_ok()
    got = xs.float().cpu()
    assert torch.allclose(got, x, atol=0.06, rtol=0.03), float((got - x).abs().max())
    if with_keep:
        m = keep[:, None, :].expand(B, C, T)
        assert torch.equal(xs.cpu()[m], cond[m])


def test_unipc_step_kernel_zero_tail_columns():
    """Action vectors padded beyond the real action width: the padding columns get no velocity and stay zero."""
    from phyai_b200.models.cosmos3.sampler_unipc import FusedUniPCStream, UniPCMultistepSampler

    g = torch.Generator().manual_seed(4)
    s = UniPCMultistepSampler()
    s.set_timesteps(3)
    a = torch.randn(2, 8, 32, generator=g).bfloat16()
    a[:, :, 7:] = 0
    xs = a.cuda().contiguous()
    st = FusedUniPCStream(s, xs, view=(1, 8, 32), live_inner=7)
    for _ in range(3):
        st.step(torch.randn(2, 8, 32, generator=g).bfloat16().cuda())
    _status_ok()
    assert float(xs[:, :, 7:].abs().max()) == 0.0 and float(xs[:, :, :7].abs().max()) > 0.0


@pytest.mark.parametrize("xdt,wdt,M,K,N", [(torch.float32, torch.float32, 1, 256, 5120), (torch.bfloat16, torch.bfloat16, 50, 7, 33),
                                           (torch.float16, torch.float16, 5, 100, 12), (torch.float32, torch.bfloat16, 9, 31, 64)])
def test_linear_simt_matches_fp32(xdt, wdt, M, K, N):
    """The CUDA-core linear that takes what the tensor-core GEMM refuses (fp32 / fp16 operands, odd K or N)."""
    from phyai_b200 import ops

    g = torch.Generator().manual_seed(7)
    x = torch.randn(M, K, generator=g).to(xdt).cuda()
    w = (torch.randn(N, K, generator=g) * 0.2).to(wdt).cuda()
    b = torch.randn(N, generator=g).to(wdt).cuda()
    y = ops.linear_simt(x, w, b)
    _status_ok()
    want = x.float() @ w.float().t() + b.float()
    assert y.dtype == xdt and y.shape == (M, N)
    tol = 1e-4 if xdt == torch.float32 else 2e-2
    assert torch.allclose(y.float(), want, atol=tol * float(want.abs().max()), rtol=tol)


def test_odd_linear_layer_runs_own_kernel():
    """A ReplicatedLinear with fp32 weights on the b200 kernel path: served by linear_simt, not by a library GEMM."""
    from phyai_b200 import ops
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.layers import linear as L
    from phyai_b200.layers.linear import ReplicatedLinear

    init_engine_config(EngineConfig(device=DeviceConfig("cuda", torch.bfloat16)))
    L.init()
    lin = ReplicatedLinear(256, 40, bias=True, params_dtype=torch.float32)
    with torch.no_grad():
        lin.weight.normal_(0, 0.1)
        lin.bias.normal_(0, 0.1)
    x = torch.randn(3, 256, device="cuda")
    c0 = ops.launch_counter()
    y, _ = lin(x)
    assert ops.launch_counter() == c0 + 1
    want = x @ lin.weight.t() + lin.bias
    assert torch.allclose(y, want, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("window,cap,D,Hq,Hkv", [(37, 0.0, 128, 4, 2), (0, 30.0, 64, 4, 4), (100, 50.0, 256, 8, 1)])
def test_attention_window_and_soft_cap(window, cap, D, Hq, Hkv):
    """Sliding window and logit soft cap in the tcgen05 latency kernel against the eager statement of the layer."""
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.layers.attention.layers import Attention

    init_engine_config(EngineConfig(device=DeviceConfig("cuda", torch.bfloat16)))
    g = torch.Generator().manual_seed(D + window)
    B, Sq, Sk = 2, 150, 333
    q = torch.randn(B, Sq, Hq, D, generator=g).bfloat16().cuda()
    k = torch.randn(B, Sk, Hkv, D, generator=g).bfloat16().cuda()
    v = torch.randn(B, Sk, Hkv, D, generator=g).bfloat16().cuda()
    layer = Attention(Hq, D, Hkv, causal=True, sliding_window=window or None, logits_soft_cap=cap or None, backend="b200")
    from phyai_b200 import ops

    c0 = ops.launch_counter()
    got = layer(q, k, v)
    assert ops.launch_counter() == c0 + 1                      # the kernel ran, not the eager statement
    _status_ok()
    want = layer._eager(q.float(), k.float(), v.float(), None)
    assert torch.allclose(got.float(), want, atol=2e-2, rtol=2e-2), float((got.float() - want).abs().max())


@pytest.mark.parametrize("M,K,N", [(50, 1024, 1024), (300, 256, 520), (7, 4096, 1024)])
def test_gemm_second_output_with_column_factor(M, K, N):
    """``out2 = out * (1 + col_scale2)`` beside a gated-residual store with row sums of squares (the producer half of
    an AdaRMS norm folded into GEMM epilogues) against fp32."""
    from phyai_b200 import ops

    g = torch.Generator().manual_seed(K + M)
    x = (torch.randn(M, K, generator=g) * 0.3).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    res = torch.randn(M, N, generator=g).bfloat16().cuda()
    gate = torch.randn(N, generator=g).bfloat16().cuda()
    cs = (torch.randn(N, generator=g) * 0.3).bfloat16().cuda()
    h = res.clone()
    ss = torch.zeros(M, dtype=torch.float32, device="cuda")
    out2 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.gemm(x, w, h, residual=h, col_gate=gate, sumsq=ss, out2=out2, col_scale2=cs)
    _status_ok()
    want_h = res.float() + (x.float() @ w.float().t()) * gate.float()
    assert torch.allclose(h.float(), want_h, atol=2e-2 * float(want_h.abs().max()), rtol=2e-2)
    hb = h.float()                                   # the second output and the sums are taken from the stored (rounded) rows
    assert torch.allclose(out2.float(), hb * (1 + cs.float()), atol=1e-2 * float(hb.abs().max()), rtol=1e-2)
    assert torch.allclose(ss, hb.pow(2).sum(-1), rtol=1e-3, atol=1e-3)


def test_domain_linear_matches_fp32():
    """Per-sample weight selection by an on-device domain id (the embodiment-specific action projections of Cosmos3)."""
    from phyai_b200 import ops

    g = torch.Generator().manual_seed(11)
    B, T, K, N, D = 3, 33, 64, 520, 5
    x = torch.randn(B, T, K, generator=g).bfloat16().cuda()
    w = (torch.randn(D, K * N, generator=g) * 0.1).bfloat16().cuda()
    bias = torch.randn(D, N, generator=g).bfloat16().cuda()
    dom = torch.tensor([4, 0, 2], dtype=torch.int64, device="cuda")
    y = ops.domain_linear(x, w, bias, dom)
    _status_ok()
    want = torch.bmm(x.float(), w[dom].float().view(B, K, N)) + bias[dom].float()[:, None]
    assert y.shape == (B, T, N)
    assert torch.allclose(y.float(), want, atol=2e-2 * float(want.abs().max()), rtol=2e-2)
