"""Offline tokenisation: text corpus -> flat little-endian uint32 token file.

    python scripts/prepare_data.py --dataset fineweb-edu --subset sample-10BT --min-score 5 --max-score 5 --out data/fw5.bin
    python scripts/prepare_data.py --dataset nemotron --subset everything --out data/nemotron.bin
    python scripts/prepare_data.py --dataset text --input corpus.txt --out data/corpus.bin     (one document per line)
    python scripts/prepare_data.py --dataset synthetic --tokens 10000000 --vocab 32000 --out data/synth.bin

The output is what ``PackedTokenDataset`` memory-maps. Documents are tokenised in batches of 2048 by a
process pool (``tiktoken`` releases the GIL but a pool also spreads the Python overhead); results are
written strictly in submission order and at most ``4 * workers`` batches are in flight, so memory stays
bounded. The file is written under a temporary name and renamed when complete, so a reader never sees
a truncated file. Reference counterpart: scripts/prepare_data.py.
"""

from __future__ import annotations

import argparse
import collections
import itertools
import os
import sys
import time
from concurrent.futures import ProcessPoolExecutor
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

DOCS_PER_BATCH = 2048


def encode_batch(job):
    texts, encoding, eot = job
    import tiktoken

    enc = tiktoken.get_encoding(encoding)
    ids: list[int] = []
    for t in texts:
        ids.extend(enc.encode_ordinary(t))
        ids.append(eot)
    return np.asarray(ids, dtype=np.uint32)


def batched(it, n):
    it = iter(it)
    while chunk := list(itertools.islice(it, n)):
        yield chunk


def text_stream(args):
    if args.dataset == "text":
        with open(args.input, encoding="utf-8") as fh:
            for line in fh:
                if line.strip():
                    yield line.rstrip("\n")
        return
    from datasets import get_dataset_config_names, load_dataset

    streaming = not args.no_streaming
    if args.dataset == "fineweb-edu":
        ds = load_dataset("HuggingFaceFW/fineweb-edu", name=args.subset, split="train", streaming=streaming)
        for row in ds:
            if args.min_score <= row.get("int_score", args.min_score) <= args.max_score and \
               row.get("token_count", args.min_token_count) >= args.min_token_count:
                yield row["text"]
    elif args.dataset == "nemotron":
        repo = "nvidia/Nemotron-Pretraining-Specialized-v1.1"
        names = get_dataset_config_names(repo) if args.subset == "everything" else [args.subset]
        for name in names:
            for row in load_dataset(repo, name=name, split="train", streaming=streaming):
                if len(row.get("text", "")) >= args.min_chars:
                    yield row["text"]
    else:
        raise ValueError(f"unknown dataset {args.dataset}")


def write_synthetic(args, tmp: Path) -> int:
    import torch

    from gdnet_b200.data.synthetic import synthetic_packed_batch

    g = torch.Generator().manual_seed(args.seed)
    done = 0
    with open(tmp, "wb") as fh:
        while done < args.tokens:
            seq, _, _ = synthetic_packed_batch(64, 16384 - 1, args.vocab, 1024.0, g)
            arr = seq.numpy().astype(np.uint32).reshape(-1)[: args.tokens - done]
            arr.tofile(fh)
            done += arr.size
    return done


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", required=True, choices=["fineweb-edu", "nemotron", "text", "synthetic"])
    ap.add_argument("--subset", default="sample-10BT")
    ap.add_argument("--encoding", default="cl100k_base")
    ap.add_argument("--out", required=True)
    ap.add_argument("--input", default="")
    ap.add_argument("--min-score", type=int, default=3)
    ap.add_argument("--max-score", type=int, default=5)
    ap.add_argument("--min-token-count", type=int, default=128)
    ap.add_argument("--min-chars", type=int, default=0)
    ap.add_argument("--workers", type=int, default=max(1, (os.cpu_count() or 2) - 1))
    ap.add_argument("--no-streaming", action="store_true")
    ap.add_argument("--tokens", type=int, default=1_000_000)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()

    out = Path(args.out)
    out.parent.mkdir(parents=True, exist_ok=True)
    tmp = out.with_suffix(out.suffix + ".partial")
    t0 = time.time()
    if args.dataset == "synthetic":
        total = write_synthetic(args, tmp)
    else:
        import tiktoken

        eot = tiktoken.get_encoding(args.encoding).eot_token
        total = 0
        pending: collections.deque = collections.deque()
        with open(tmp, "wb") as fh, ProcessPoolExecutor(args.workers) as pool:
            def drain(limit: int) -> None:
                nonlocal total
                while len(pending) > limit:
                    arr = pending.popleft().result()     # oldest first: output order = input order
                    arr.tofile(fh)
                    total += arr.size

            for docs in batched(text_stream(args), DOCS_PER_BATCH):
                pending.append(pool.submit(encode_batch, (docs, args.encoding, eot)))
                drain(4 * args.workers)
            drain(0)
    os.replace(tmp, out)
    print(f"[prepare] {total:,} tokens -> {out} ({out.stat().st_size / 2**30:.2f} GiB) in {time.time() - t0:.0f} s")


if __name__ == "__main__":
    main()
