"""FLOP and minimum-traffic models of the served models, stage by stage.

Every stage is described by its matrix products ``(rows, out_features, in_features)`` and attention calls
``(query_rows, kv_rows, heads, head_dim)``; FLOPs are ``2 m n k`` per product and ``4 q kv h d`` per attention
call; the traffic floor is every weight read once plus the activations entering and leaving each product
(bf16). A stage's roofline time is ``max(flops / peak_flops, bytes / peak_bandwidth)``.
Reference counterparts: benchmark/pi05/model_flops.py:11-265, benchmark/cosmos3_policy/model_flops_cosmos3.py.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class Stage:
    name: str
    gemms: list[tuple[int, int, int, int]] = field(default_factory=list)       # (count, m, n, k)
    attns: list[tuple[int, int, int, int, int]] = field(default_factory=list)  # (count, q, kv, heads, head_dim)
    extra_bytes: int = 0                                                       # KV reads and the like

    def gemm(self, m: int, n: int, k: int, count: int = 1) -> "Stage":
        self.gemms.append((count, m, n, k))
        return self

    def attn(self, q: int, kv: int, heads: int, head_dim: int, count: int = 1, kv_heads: int | None = None) -> "Stage":
        self.attns.append((count, q, kv, heads, head_dim))
        self.extra_bytes += count * 2 * kv * (kv_heads or heads) * head_dim * 2     # K and V read once
        return self

    @property
    def flops(self) -> float:
        return float(sum(c * 2 * m * n * k for c, m, n, k in self.gemms) + sum(c * 4 * q * kv * h * d for c, q, kv, h, d in self.attns))

    @property
    def weight_bytes(self) -> float:
        return float(sum(c * n * k * 2 for c, _, n, k in self.gemms))

    @property
    def bytes(self) -> float:
        act = sum(c * (m * k + m * n) * 2 for c, m, n, k in self.gemms)
        return self.weight_bytes + act + self.extra_bytes

    def roofline_ms(self, peaks: dict, sustained: bool = True) -> float:
        tf = peaks["bf16_tflops_sustained" if sustained and "bf16_tflops_sustained" in peaks else "bf16_tflops"]
        return max(self.flops / (tf * 1e9), self.bytes / (peaks["hbm_gbs"] * 1e6))

    def bound(self, peaks: dict) -> str:
        tf = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        return "compute" if self.flops / (tf * 1e9) >= self.bytes / (peaks["hbm_gbs"] * 1e6) else "memory"


def pi05_stages(cfg, batch: int = 1, num_images: int = 3, lang_tokens: int = 48) -> list[Stage]:
    """Vision tower, prefix decoder and action expert of Pi0.5 (``cfg`` is a ``PI05Config``)."""
    v, t, e = cfg.vision, cfg.text, cfg.expert
    patches = (v.image_size // v.patch_size) ** 2
    mv = batch * num_images * patches
    hd_v = v.hidden_size // v.num_attention_heads
    vision = Stage("vision")
    vision.gemm(mv, v.hidden_size, v.num_channels * v.patch_size ** 2)
    L = v.num_hidden_layers
    vision.gemm(mv, 3 * v.hidden_size, v.hidden_size, L).gemm(mv, v.hidden_size, v.hidden_size, L)
    vision.gemm(mv, v.intermediate_size, v.hidden_size, L).gemm(mv, v.hidden_size, v.intermediate_size, L)
    vision.attn(patches, patches, v.num_attention_heads, hd_v, L * batch * num_images)
    vision.gemm(mv, v.projection_dim, v.hidden_size)

    per = num_images * patches + lang_tokens
    mp = batch * per
    qkv = (t.num_attention_heads + 2 * t.num_key_value_heads) * t.head_dim
    prefix = Stage("prefix")
    L = t.num_hidden_layers
    prefix.gemm(mp, qkv, t.hidden_size, L)
    # the last block only produces K / V: no attention, output projection or MLP
    prefix.gemm(mp, t.hidden_size, t.num_attention_heads * t.head_dim, L - 1)
    prefix.gemm(mp, 2 * t.intermediate_size, t.hidden_size, L - 1).gemm(mp, t.hidden_size, t.intermediate_size, L - 1)
    prefix.attn(per, per, t.num_attention_heads, t.head_dim, (L - 1) * batch, kv_heads=t.num_key_value_heads)

    me = batch * cfg.chunk_size
    steps = cfg.num_inference_steps
    expert = Stage("expert")
    L = e.num_hidden_layers
    expert.gemm(me, e.hidden_size, cfg.max_action_dim, steps).gemm(me, cfg.max_action_dim, e.hidden_size, steps)
    expert.gemm(me, qkv, e.hidden_size, L * steps).gemm(me, e.hidden_size, t.num_attention_heads * t.head_dim, L * steps)
    expert.gemm(me, 2 * e.intermediate_size, e.hidden_size, L * steps).gemm(me, e.hidden_size, e.intermediate_size, L * steps)
    expert.attn(cfg.chunk_size, per + cfg.chunk_size, t.num_attention_heads, t.head_dim, L * steps * batch,
                kv_heads=t.num_key_value_heads)
    return [vision, prefix, expert]


def cosmos3_step_stages(cfg, gen_tokens: int, text_tokens: int, batch: int = 1, guided: bool = True) -> list[Stage]:
    """One denoise step of the Cosmos3 generation tower (``cfg`` is a ``Cosmos3Config``): with guidance the
    conditional and unconditional passes both run."""
    passes = 2 if guided else 1
    H, L = cfg.hidden_size, cfg.num_hidden_layers
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    m = batch * gen_tokens
    gen = Stage("gen_tower_step")
    c = L * passes
    gen.gemm(m, (hq + 2 * hkv) * d, H, c).gemm(m, H, hq * d, c)
    gen.gemm(m, 2 * cfg.intermediate_size, H, c).gemm(m, H, cfg.intermediate_size, c)
    gen.attn(gen_tokens, gen_tokens + text_tokens, hq, d, c * batch, kv_heads=hkv)
    return [gen]


def report(stages: list[Stage], measured_ms: dict[str, float], peaks: dict) -> list[dict]:
    """Join measured stage latencies with the model: one row per stage plus the fraction of roofline."""
    rows = []
    for s in stages:
        ms = measured_ms.get(s.name)
        roof = s.roofline_ms(peaks)
        rows.append({"stage": s.name, "gflop": round(s.flops / 1e9, 2), "weights_mb": round(s.weight_bytes / 1e6, 1),
                     "traffic_mb": round(s.bytes / 1e6, 1), "bound": s.bound(peaks), "roofline_ms": round(roof, 4),
                     "measured_ms": None if ms is None else round(ms, 4),
                     "frac_of_roofline": None if not ms else round(roof / ms, 3),
                     "tflops": None if not ms else round(s.flops / ms / 1e9, 1),
                     "gbs": None if not ms else round(s.bytes / ms / 1e6, 1)})
    return rows


def to_markdown(rows: list[dict]) -> str:
    cols = ["stage", "gflop", "weights_mb", "traffic_mb", "bound", "roofline_ms", "measured_ms", "frac_of_roofline", "tflops", "gbs"]
    out = ["| " + " | ".join(cols) + " |", "|" + "---|" * len(cols)]
    out += ["| " + " | ".join("–" if r[c] is None else str(r[c]) for c in cols) + " |" for r in rows]
    return "\n".join(out)


def to_svg(rows: list[dict], title: str, width: int = 640) -> str:
    """Horizontal bars, measured against roofline, as a dependency-free SVG (no plotting library needed)."""
    rows = [r for r in rows if r["measured_ms"]]
    top = max(r["measured_ms"] for r in rows) if rows else 1.0
    h = 40 + 46 * len(rows)
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{h}" font-family="monospace" font-size="12">',
             f'<text x="8" y="18">{title}</text>']
    for i, r in enumerate(rows):
        y = 34 + 46 * i
        wm = (width - 200) * r["measured_ms"] / top
        wr = (width - 200) * r["roofline_ms"] / top
        parts += [f'<text x="8" y="{y + 14}">{r["stage"]}</text>',
                  f'<rect x="120" y="{y}" width="{wm:.1f}" height="14" fill="#4477aa"/>',
                  f'<rect x="120" y="{y + 16}" width="{wr:.1f}" height="14" fill="#ccbb44"/>',
                  f'<text x="{124 + wm:.1f}" y="{y + 12}">{r["measured_ms"]} ms measured</text>',
                  f'<text x="{124 + wr:.1f}" y="{y + 28}">{r["roofline_ms"]} ms roofline ({r["bound"]})</text>']
    parts.append("</svg>")
    return "\n".join(parts)


__all__ = ["Stage", "pi05_stages", "cosmos3_step_stages", "report", "to_markdown", "to_svg"]
