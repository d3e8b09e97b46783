"""Serve Pi0 on one GPU (state enters as a vector; 48-token prompt).

    python examples/pi0/run_pi0.py [--checkpoint DIR]
"""

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import torch  # noqa: E402

from phyai_b200.engine import Engine, EngineArgs  # noqa: E402
from phyai_b200.engine_config import DeviceConfig, EngineConfig  # noqa: E402
from phyai_b200.models.pi0.main_pi0 import PI0Args  # noqa: E402
from phyai_b200.models.pi0.scheduler_ws1_pi0 import PI0Request  # noqa: E402
from phyai_b200.tools.pi0 import PI0Processor  # noqa: E402
from phyai_b200.tools.tokenizer import ByteTokenizer  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", default=None)
    a = ap.parse_args()
    dev = "cuda:0"
    engine = Engine(EngineArgs("pi0", PI0Args(checkpoint_dir=a.checkpoint, max_batch_size=1, inputs_image_shape=[[224, 224, 3]] * 3),
                               EngineConfig(device=DeviceConfig(dev, torch.bfloat16))))
    proc = PI0Processor(tokenizer=ByteTokenizer(), device=dev, action_dim=7)
    inp = proc.preprocess({"images": [torch.rand(1, 3, 224, 224)] * 3, "state": torch.rand(1, 8), "task": "open the drawer"})
    out = engine.step(PI0Request(inp.pixel_values, inp.input_ids, inp.lang_lens, inp.state, torch.randn(1, 50, 32, device=dev, dtype=torch.bfloat16)))
    print("action chunk", tuple(proc.postprocess(out).shape))
    engine.close()


if __name__ == "__main__":
    main()
