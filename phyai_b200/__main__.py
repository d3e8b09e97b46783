"""``python -m phyai_b200 show-env``: one page about the installation (versions, toolchain, built extensions, JIT cache,
every ``PHYAI_*`` switch with its current value). Counterpart of ``python -m phyai_kernel show-env`` in the reference
(phyai-kernel/phyai_kernel/__main__.py)."""

from __future__ import annotations

import json
import os
import shutil
import sys
from pathlib import Path


def show_env() -> dict:
    import torch

    from . import jit
    from .env import envs

    root = Path(__file__).resolve().parent
    info: dict = {
        "python": sys.version.split()[0],
        "torch": torch.__version__,
        "torch_cuda": torch.version.cuda,
        "nvcc": shutil.which("nvcc") or str(Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"),
        "extensions": {p.name: p.stat().st_size for p in sorted(root.glob("_*.so"))},
        "jit_cache_dir": str(jit.cache_dir()),
        "cuda_available": torch.cuda.is_available(),
        "env": {name: {"value": f.get(), "set": f.is_set()} for name, f in sorted(envs.fields().items())},
    }
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        info["gpu"] = {"name": p.name, "sm": f"{p.major}{p.minor}", "sms": p.multi_processor_count,
                       "memory_gib": round(p.total_memory / 2 ** 30, 1), "count": torch.cuda.device_count()}
    return info


def main(argv: list[str] | None = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if argv[:1] != ["show-env"]:
        print("usage: python -m phyai_b200 show-env", file=sys.stderr)
        return 2
    print(json.dumps(show_env(), indent=1, default=str))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
