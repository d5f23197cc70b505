"""ms/step of a small GDNet in fp32, bf16 and fp8 on one GPU (reference: scripts/fp8_profile.py).

    python scripts/fp8_profile.py [--d 1024] [--layers 4] [--batch 4] [--seq 2048] [--steps 10]
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdnet_b200.loss import projected_step  # noqa: E402
from gdnet_b200.model import GDNet  # noqa: E402
from gdnet_b200.utils.fp8 import cast_for_precision  # noqa: E402


def run(precision, args):
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(0)
    model = GDNet(vocab_size=32000, d_embed=args.d, d=args.d, n_layers=args.layers, n_cycles=2, kernel_size=4,
                  chunk_size=args.seq).to(dev)
    cast_for_precision(model, precision)
    if dev.type == "cuda" and precision != "fp32":
        from gdnet_b200.train.engine import TrainEngine

        runner, params, opt = TrainEngine(model, precision=precision), None, None
    else:
        runner, params = model, list(model.parameters())
        opt = torch.optim.AdamW(params, lr=1e-3)
    tok = torch.randint(0, 32000, (args.batch, args.seq), device=dev)
    tgt = torch.randint(0, 32000, (args.batch, args.seq), device=dev)
    for _ in range(3):
        projected_step(runner, params, opt, tok, tgt, precision=precision)
    if dev.type == "cuda":
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    for _ in range(args.steps):
        loss = projected_step(runner, params, opt, tok, tgt, precision=precision)
    ms = float("nan")
    if dev.type == "cuda":
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
    print(f"{precision:>5}: {ms:9.2f} ms/step  {args.batch * args.seq / ms * 1000:12,.0f} tok/s  loss {float(loss):.3f}")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--d", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=10)
    a = ap.parse_args()
    for p in ("fp32", "bf16", "fp8"):
        run(p, a)
