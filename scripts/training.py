"""GDNet pre-training (reference entry point: scripts/training.py).

    python scripts/training.py --config configs/training.yaml
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 scripts/training.py --config ...
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdnet_b200.config import Config  # noqa: E402
from gdnet_b200.train.trainer import train  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="configs/training.yaml")
    ap.add_argument("--no-shell", action="store_true", help="do not start the interactive prompt on rank 0")
    args = ap.parse_args()
    state = train(Config.from_yaml(args.config), interactive=not args.no_shell)
    print(f"finished at step {state.step}: loss {state.loss:.4f}, {state.tok_per_sec:,.0f} tok/s")


if __name__ == "__main__":
    main()
