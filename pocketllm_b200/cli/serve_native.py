"""Launcher of the native OpenAI server under tensor parallelism: starts one `pocket_engine --serve` process per rank
(rank 0 listens, the others replay its commands), waits for the listening line and forwards signals.
Role of the reference's scripts/run_cpp_serve_tp4.sh, for any rank count.

    python -m pocketllm_b200.cli.serve_native --ckpt DIR --tp 4 --port 8000 --tokenizer hf:DIR [--qwen-mtp] [--kv-cache-dtype fp8]
    python -m pocketllm_b200.cli.serve_native --benchmark-27b --random-init 0 --tp 8      # shape-only smoke server
"""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import tempfile
from pathlib import Path

BINARY = Path(__file__).resolve().parent.parent / "_C" / "pocket_engine"


def build_commands(args: argparse.Namespace, passthrough: list[str], rendezvous: str) -> list[list[str]]:
    """The command line of every rank (exposed for tests: nothing is started here)."""
    cmds = []
    for r in range(args.tp):
        c = [str(BINARY), "--serve", "--tp-world", str(args.tp), "--tp-rank", str(r), "--device", str(args.first_device + r),
             "--nccl-id-path", rendezvous, "--max-context", str(args.max_context), "--prefill-chunk-tokens", str(args.prefill_chunk)]
        if args.ckpt:
            c += ["--ckpt", args.ckpt]
        if r == 0:
            c += ["--host", args.host, "--port", str(args.port), "--model-name", args.model_name, "--tokenizer", args.tokenizer,
                  "--chat-format", args.chat_format, "--sidecar-python", sys.executable]
        cmds.append(c + passthrough)
    return cmds


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ckpt", default="")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--first-device", type=int, default=0)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--model-name", default="pocketllm-b200")
    ap.add_argument("--tokenizer", default="chars")
    ap.add_argument("--chat-format", default="qwen")
    ap.add_argument("--max-context", type=int, default=8192)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--dry-run", action="store_true", help="print the per-rank command lines and exit")
    args, passthrough = ap.parse_known_args(argv)      # everything else goes to pocket_engine unchanged
    if args.tp < 1 or args.tp > 8:
        ap.error("--tp must be 1..8")
    rendezvous = os.path.join(tempfile.mkdtemp(prefix="pocket_serve_"), "rdv")
    cmds = build_commands(args, passthrough, rendezvous)
    if args.dry_run:
        for c in cmds:
            print(" ".join(c))
        return 0
    if not BINARY.exists():
        print(f"{BINARY} is not built: run `python -m pocketllm_b200.build`", file=sys.stderr)
        return 2
    env = dict(os.environ, PYTHONPATH=str(BINARY.parent.parent.parent) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    procs = [subprocess.Popen(c, env=env) for c in reversed(cmds)]      # workers first, the listener last

    def stop(*_):
        for p in procs:
            if p.poll() is None:
                p.terminate()

    signal.signal(signal.SIGINT, stop)
    signal.signal(signal.SIGTERM, stop)
    rc = procs[-1].wait()                # rank 0
    stop()
    for p in procs:
        try:
            p.wait(timeout=30)
        except subprocess.TimeoutExpired:
            p.kill()
    return rc


if __name__ == "__main__":
    raise SystemExit(main())
