"""One command: tokenise the first phase, start training, tokenise later phases in the background.

    python scripts/run.py [--config configs/training.yaml] [--gpus N] [--data-dir data/tokenized]
                          [--skip-prepare] [--prepare-only] [--no-streaming] [--resume CKPT]

Each phase of the config gets a token-file path derived from its dataset settings. The trainer is
launched with ``python -m torch.distributed.run`` (one process per GPU, rendezvous on 127.0.0.1) on a
temporary copy of the config that carries those paths; it waits at a phase boundary until that phase's
file exists. SIGINT/SIGTERM are forwarded to the trainer, whose exit code becomes this script's.
Reference counterpart: scripts/run.py.
"""

from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import tempfile
import threading
from pathlib import Path

import yaml

ROOT = Path(__file__).resolve().parent.parent


def phase_file(phase: dict, data_dir: Path) -> str | None:
    kind = phase.get("dataset", "fineweb-edu")
    if kind == "fineweb-edu":
        sub = str(phase.get("subset", "sample-10BT")).replace("/", "_")
        return str(data_dir / f"fineweb_edu_{sub}_{phase.get('min_int_score', 3)}_{phase.get('max_int_score', 5)}.bin")
    if kind == "nemotron":
        return str(data_dir / f"nemotron_{str(phase.get('subset', 'everything')).replace('/', '_')}.bin")
    return None


def tokenise_command(phase: dict, encoding: str, no_streaming: bool) -> list[str]:
    kind = phase.get("dataset", "fineweb-edu")
    cmd = [sys.executable, str(ROOT / "scripts" / "prepare_data.py"), "--dataset", kind, "--encoding", encoding,
           "--out", phase["path"]]
    if kind == "fineweb-edu":
        cmd += ["--subset", str(phase.get("subset", "sample-10BT")), "--min-score", str(phase.get("min_int_score", 3)),
                "--max-score", str(phase.get("max_int_score", 5)),
                "--min-token-count", str(phase.get("min_token_count", 128))]
    elif kind == "nemotron":
        cmd += ["--subset", str(phase.get("subset", "everything")), "--min-chars", str(phase.get("min_chars", 0))]
    return cmd + (["--no-streaming"] if no_streaming else [])


def tokenise_phase(phase: dict, encoding: str, no_streaming: bool) -> bool:
    path = phase.get("path")
    if not path:
        return True
    p = Path(path)
    if p.exists() and p.stat().st_size > 0:
        print(f"[data] found {path} ({p.stat().st_size / 2**30:.2f} GiB)", flush=True)
        return True
    print(f"[data] tokenising -> {path}", flush=True)
    rc = subprocess.run(tokenise_command(phase, encoding, no_streaming)).returncode
    if rc != 0 or not p.exists() or p.stat().st_size == 0:
        p.unlink(missing_ok=True)            # never leave an empty or broken file for the trainer to map
        print(f"[data] tokenising {path} failed (exit {rc})", flush=True)
        return False
    return True


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=str(ROOT / "configs" / "training.yaml"))
    ap.add_argument("--gpus", type=int, default=0, help="0 = all visible GPUs")
    ap.add_argument("--data-dir", default=str(ROOT / "data" / "tokenized"))
    ap.add_argument("--skip-prepare", action="store_true")
    ap.add_argument("--prepare-only", action="store_true")
    ap.add_argument("--no-streaming", action="store_true")
    ap.add_argument("--resume", default=None)
    ap.add_argument("--master-port", type=int, default=29511)
    args = ap.parse_args()

    cfg = yaml.safe_load(open(args.config)) or {}
    data_dir = Path(args.data_dir)
    data_dir.mkdir(parents=True, exist_ok=True)
    phases = cfg.get("phases") or []
    for ph in phases:
        if not ph.get("path"):
            derived = phase_file(ph, data_dir)
            if derived:
                ph["path"] = derived
    if args.resume:
        cfg["resume"] = args.resume
    encoding = cfg.get("tokenizer", "cl100k_base")

    if not args.skip_prepare and phases:
        if not tokenise_phase(phases[0], encoding, args.no_streaming):
            return 1
    if args.prepare_only:
        ok = all(tokenise_phase(ph, encoding, args.no_streaming) for ph in phases[1:])
        return 0 if ok else 1

    with tempfile.NamedTemporaryFile("w", suffix=".yaml", delete=False) as fh:
        yaml.safe_dump(cfg, fh)
        run_cfg = fh.name

    import torch

    gpus = args.gpus or max(torch.cuda.device_count(), 1)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
           "--master-addr", "127.0.0.1", "--master-port", str(args.master_port),
           str(ROOT / "scripts" / "training.py"), "--config", run_cfg, "--no-shell"]
    child = subprocess.Popen(cmd)

    def forward(sig, _frame):
        if child.poll() is None:
            child.send_signal(sig)

    signal.signal(signal.SIGINT, forward)
    signal.signal(signal.SIGTERM, forward)
    if not args.skip_prepare and len(phases) > 1:
        threading.Thread(target=lambda: [tokenise_phase(ph, encoding, args.no_streaming) for ph in phases[1:]],
                         daemon=True).start()
    rc = child.wait()
    os.unlink(run_cfg)
    return rc


if __name__ == "__main__":
    sys.exit(main())
