"""In-process metrics: counters, gauges and latency histograms, dumpable as JSON (or Prometheus text).

The reference has logging only (phyai/src/phyai/utils/logging.py:25-71) and a JSONL bench record
(benchmark/bench_n_batch.py:84-111); serving needs per-stage latency, graph-replay counts,
plan-cache hit rates and communication bytes without a profiler attached.
"""

from __future__ import annotations

import bisect
import json
import threading
import time
from contextlib import contextmanager
from pathlib import Path

_DEFAULT_BOUNDS_MS = (0.05, 0.1, 0.25, 0.5, 1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 5000)


class Histogram:
    def __init__(self, bounds=_DEFAULT_BOUNDS_MS, keep: int = 4096) -> None:
        self.bounds = tuple(float(b) for b in bounds)
        self.buckets = [0] * (len(self.bounds) + 1)
        self.count, self.total, self.min, self.max = 0, 0.0, float("inf"), 0.0
        self._ring: list[float] = []
        self._keep, self._pos = keep, 0

    def observe(self, v: float) -> None:
        v = float(v)
        self.buckets[bisect.bisect_left(self.bounds, v)] += 1
        self.count += 1
        self.total += v
        self.min, self.max = min(self.min, v), max(self.max, v)
        if len(self._ring) < self._keep:
            self._ring.append(v)
        else:
            self._ring[self._pos] = v
            self._pos = (self._pos + 1) % self._keep

    def quantile(self, q: float) -> float:
        """Over the most recent ``keep`` observations."""
        if not self._ring:
            return float("nan")
        s = sorted(self._ring)
        k = (len(s) - 1) * q
        lo, hi = int(k), min(int(k) + 1, len(s) - 1)
        return s[lo] + (s[hi] - s[lo]) * (k - lo)

    def snapshot(self) -> dict:
        return {"count": self.count, "sum": self.total, "min": None if self.count == 0 else self.min, "max": self.max,
                "mean": self.total / self.count if self.count else None, "p50": self.quantile(0.5), "p90": self.quantile(0.9),
                "p99": self.quantile(0.99), "buckets": dict(zip([*map(str, self.bounds), "+Inf"], self.buckets))}


class MetricsRegistry:
    def __init__(self) -> None:
        self._lock = threading.Lock()
        self.counters: dict[str, float] = {}
        self.gauges: dict[str, float] = {}
        self.histograms: dict[str, Histogram] = {}

    def inc(self, name: str, by: float = 1.0) -> None:
        with self._lock:
            self.counters[name] = self.counters.get(name, 0.0) + by

    def set(self, name: str, value: float) -> None:
        with self._lock:
            self.gauges[name] = float(value)

    def observe(self, name: str, value: float, bounds=_DEFAULT_BOUNDS_MS) -> None:
        with self._lock:
            h = self.histograms.get(name)
            if h is None:
                h = self.histograms[name] = Histogram(bounds)
            h.observe(value)

    @contextmanager
    def timer(self, name: str):
        """Wall-clock milliseconds of the block (host side; pair with CUDA events for device time)."""
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.observe(name, (time.perf_counter() - t0) * 1e3)

    def hit_rate(self, hits: str, misses: str) -> float | None:
        h, m = self.counters.get(hits, 0.0), self.counters.get(misses, 0.0)
        return h / (h + m) if h + m else None

    def snapshot(self) -> dict:
        with self._lock:
            return {"counters": dict(self.counters), "gauges": dict(self.gauges),
                    "histograms": {k: v.snapshot() for k, v in self.histograms.items()}}

    def dump(self, path: str | Path) -> Path:
        p = Path(path)
        p.write_text(json.dumps(self.snapshot(), indent=2))
        return p

    def prometheus_text(self, prefix: str = "phyai_b200") -> str:
        clean = lambda s: "".join(c if c.isalnum() else "_" for c in s)  # noqa: E731
        out = []
        snap = self.snapshot()
        for k, v in snap["counters"].items():
            out += [f"# TYPE {prefix}_{clean(k)} counter", f"{prefix}_{clean(k)} {v}"]
        for k, v in snap["gauges"].items():
            out += [f"# TYPE {prefix}_{clean(k)} gauge", f"{prefix}_{clean(k)} {v}"]
        for k, h in snap["histograms"].items():
            n, acc = f"{prefix}_{clean(k)}", 0
            out.append(f"# TYPE {n} histogram")
            for b, c in h["buckets"].items():
                acc += c
                out.append(f'{n}_bucket{{le="{b}"}} {acc}')
            out += [f"{n}_sum {h['sum']}", f"{n}_count {h['count']}"]
        return "\n".join(out) + "\n"

    def reset(self) -> None:
        with self._lock:
            self.counters.clear(), self.gauges.clear(), self.histograms.clear()


_REGISTRY = MetricsRegistry()


def metrics() -> MetricsRegistry:
    return _REGISTRY


__all__ = ["Histogram", "MetricsRegistry", "metrics"]
