"""Serve Pi0.5 on one GPU: raw observation -> processor -> engine -> un-normalised action chunk.

    python examples/pi05/run_pi05.py [--checkpoint DIR] [--steps 20]

Without ``--checkpoint`` the model runs with random weights at the pi05_base geometry (latency is
the same; the actions are noise) and a byte-level stand-in tokenizer.
"""

import argparse
import statistics
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import torch  # noqa: E402

from phyai_b200.engine import Engine, EngineArgs  # noqa: E402
from phyai_b200.engine_config import DeviceConfig, EngineConfig  # noqa: E402
from phyai_b200.models.pi05.main_pi05 import PI05Args  # noqa: E402
from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request  # noqa: E402
from phyai_b200.tools.pi05 import PI05Processor  # noqa: E402
from phyai_b200.tools.tokenizer import ByteTokenizer, get_tokenizer  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--tokenizer", default=None, help="tokenizer directory (default: byte-level stand-in)")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--task", default="pick up the red block")
    a = ap.parse_args()
    dev = "cuda:0"
    engine = Engine(EngineArgs("pi05", PI05Args(checkpoint_dir=a.checkpoint, max_batch_size=1, inputs_image_shape=[[224, 224, 3]] * 3),
                               EngineConfig(device=DeviceConfig(dev, torch.bfloat16))))
    tok = get_tokenizer(a.tokenizer) if a.tokenizer else ByteTokenizer()
    proc = (PI05Processor.from_pretrained(a.checkpoint, tokenizer=tok, device=dev, action_dim=7) if a.checkpoint and (Path(a.checkpoint) / "policy_preprocessor.json").is_file()
            else PI05Processor(tokenizer=tok, device=dev, action_dim=7))
    obs = {"images": [torch.rand(1, 3, 480, 640) for _ in range(3)], "state": torch.rand(1, 8) * 2 - 1, "task": [a.task]}
    lat = []
    for i in range(a.steps):
        inp = proc.preprocess(dict(obs))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        chunk = engine.step(PI05Request(pixel_values=inp.pixel_values, input_ids=inp.input_ids, lang_lens=inp.lang_lens,
                                        noise=torch.randn(1, 50, 32, device=dev, dtype=torch.bfloat16)))
        e1.record()
        e1.synchronize()
        lat.append(e0.elapsed_time(e1))
        action = proc.postprocess(chunk)
    print(f"action chunk {tuple(action.shape)}; engine.step median {statistics.median(lat[2:]):.2f} ms over {len(lat) - 2} steps")
    engine.close()


if __name__ == "__main__":
    main()
