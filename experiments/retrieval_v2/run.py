"""Retrieval, second version: the blend gate sees how sure the retrieval was.

    python experiments/retrieval_v2/run.py [--epochs 60] [--device cpu] [--out curves.json]

In the first version (``experiments/retrieval/run.py``) nothing told the model that a key was missing: in
condition 3 the retrieval weights were diffuse but the blend gate R opened as far as for a hit. Here the
normalised retrieval entropy ``H(w) / log(n_slots)`` is one more input of the gate MLP, condition 3 carries
the value inside the query chunk (so the right answer is available locally and the memory should be ignored),
and training uses all three conditions in equal parts (reference: experiments/retrieval_v2/run.py:137-186,
260-300; it reports accuracy 1.000 on all three with R about 0.40 and H 0.08 / 0.10 / 0.16). The gate
input of the full model's ``Memory`` is built the same way.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(_HERE), "retrieval"))

import run as base          # noqa: E402  (the shared harness of experiments/retrieval)
from dataset import N_VALUES, VOCAB_SIZE  # noqa: E402
from model import RetrievalModel  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    base.add_common_args(ap)
    ap.add_argument("--no-entropy-gate", action="store_true", help="ablation: train on the same data without the entropy input")
    args = ap.parse_args()
    torch.manual_seed(args.seed)
    model = RetrievalModel(VOCAB_SIZE, N_VALUES, base.D, base.D_SIG, base.D_C, args.n_slots, base.N_LAYERS,
                           base.KERNEL_SIZE, base.N_CYCLES, use_pos_gate=True, entropy_gate=not args.no_entropy_gate)
    train = base.make_sets(args, (1, 2, 3), args.n_train // 3, 0, value_in_query=True)
    val = base.make_sets(args, (1, 2, 3), args.n_val, 10, value_in_query=True)
    hist = base.fit(model, train, val, args)
    base.save_curves({"PosGateCAM+entropy": hist}, args.out)


if __name__ == "__main__":
    main()
