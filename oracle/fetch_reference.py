"""Places an UNMODIFIED working copy of the reference under ``oracle/_ref/`` (test infrastructure).

    python oracle/fetch_reference.py [--source DIR]

The reference is pure Python (Triton kernels inside Python files), so nothing is compiled: the recipe
copies the files the hot path, its two callers and the small trainer consist of, byte for byte, from a
checkout of djo1996/Palimpsa (``--source``, default ``$PALIMPSA_REFERENCE``, else a folder named ``reference``
beside this repository):

    palimpsa/                    ops (Triton chunk / fused-recurrent kernels, ``palimpsa_ref``), layers, models
    train_nano.py                the character-level trainer (train_nano.py:1-185)
    data/shakespeare_char/       its corpus and tokeniser script
    config/palimpsa_170M.json    the 170M model's shape (for a packed variable-length model step)

and then runs the copied ``data/shakespeare_char/prepare.py`` once so that ``train.bin`` / ``val.bin`` /
``meta.pkl`` exist beside it (the script finds ``input.txt`` and downloads nothing).

``oracle/_ref/`` is ignored by git: reference sources never enter this repository's history.  The copy is
used by GPU tests (parity and speed of the CUDA ops against the reference's own Triton kernels on the same
device; the reference's layer and trainer running on top of the CUDA ops) and by ``bench.py``'s
``gpu_baseline`` figure.  Nothing under ``palimpsa_b200/`` imports it, and every user skips or reports
"unavailable" when the folder is absent.
"""
from __future__ import annotations

import argparse
import filecmp
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
TREES = ("palimpsa",)
FILES = ("train_nano.py", "data/shakespeare_char/input.txt", "data/shakespeare_char/prepare.py",
         "config/palimpsa_170M.json")


def default_source() -> str:
    return os.environ.get("PALIMPSA_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def available() -> bool:
    """True when the copy is in place (ops, layer, trainer and tokenised corpus)."""
    need = ("palimpsa/ops/palimpsa/chunk_palimpsa_forgetting_scalar.py",
            "palimpsa/ops/palimpsa/fused_recurrent_palimpsa.py", "palimpsa/layers/palimpsa.py", "train_nano.py",
            "data/shakespeare_char/train.bin")
    return all(os.path.exists(os.path.join(DEST, n)) for n in need)


def _make_writable(tree: str) -> None:
    for d, _, files in os.walk(tree):
        os.chmod(d, 0o755)
        for f in files:
            os.chmod(os.path.join(d, f), 0o644)


def fetch(source: str | None = None, verbose: bool = False) -> bool:
    """Copies the files; returns False (and touches nothing) when the source checkout is absent."""
    source = source or default_source()
    if not os.path.isdir(os.path.join(source, "palimpsa", "ops", "palimpsa")):
        if verbose:
            print(f"reference checkout not found at {source}; oracle/_ref left as it is")
        return False
    os.makedirs(DEST, exist_ok=True)
    for tree in TREES:
        dst = os.path.join(DEST, tree)
        if os.path.isdir(dst):
            _make_writable(dst)
            shutil.rmtree(dst)
        shutil.copytree(os.path.join(source, tree), dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"),
                        copy_function=shutil.copyfile)
        _make_writable(dst)                                # a read-only checkout must not make the copy read-only
    for rel in FILES:
        dst = os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(source, rel), dst)
    for rel in FILES:                                      # byte-for-byte: the copy is the reference, unmodified
        assert filecmp.cmp(os.path.join(source, rel), os.path.join(DEST, rel), shallow=False), rel
    data = os.path.join(DEST, "data", "shakespeare_char")
    if not os.path.exists(os.path.join(data, "train.bin")):
        subprocess.run([sys.executable, os.path.join(data, "prepare.py")], check=True, cwd=data,
                       stdout=None if verbose else subprocess.DEVNULL)
    if verbose:
        print("reference copied to", DEST)
    return True


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=None)
    a = ap.parse_args()
    sys.exit(0 if fetch(a.source, verbose=True) else 1)
