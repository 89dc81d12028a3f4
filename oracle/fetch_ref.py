"""Fetches the reference's own CPU LoRA worker for the timed CPU baseline.  TEST/BENCH INFRASTRUCTURE.

    python oracle/fetch_ref.py [--reference <reference checkout>]

Copies ``lora_cpu/lora_shm_op/app.py`` of the reference checkout, unmodified, to
``oracle/_ref/app.py``.  That folder is ignored by git (no reference source enters the history)
but travels with the working tree to the machine that runs the benchmark, where the reference
checkout itself is not mounted.  ``bench.py``'s CPU legs drive this file's ``LoRAapp.run`` worker
processes over real shared memory (``oracle/ref_worker_baseline.py``); without the copy they fall
back to the oracle's restatement of the same arithmetic and say so (``kind: "port"``).
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = [("lora_cpu/lora_shm_op/app.py", "app.py")]


def fetch(reference: str) -> bool:
    """Returns True when every file was copied; False (and copies nothing) when the checkout is absent."""
    srcs = [os.path.join(reference, rel) for rel, _ in FILES]
    if not all(os.path.isfile(s) for s in srcs):
        return False
    os.makedirs(DEST, exist_ok=True)
    for src, (_, name) in zip(srcs, FILES):
        shutil.copyfile(src, os.path.join(DEST, name))
    with open(os.path.join(DEST, "SOURCE.txt"), "w") as f:
        for src, (rel, name) in zip(srcs, FILES):
            digest = hashlib.sha256(open(src, "rb").read()).hexdigest()
            f.write(f"{name}  <-  {rel}  sha256 {digest}\n")
    return True


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("REFERENCE_ROOT", "/root/reference"))
    args = ap.parse_args()
    ok = fetch(args.reference)
    print("fetched into", DEST if ok else "(nothing: no reference checkout at %s)" % args.reference)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
