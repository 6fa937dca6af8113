"""Stages the reference's own pure-Python package for the timed CPU baseline.  TEST INFRASTRUCTURE ONLY.

    python oracle/stage_ref.py [reference root]

The reference's KV-cache path on the CPU is pure Python over torch (pace/llm/cache.py,
pace/ops/attention.py, pace/ops/backends/native.py): it needs no compiled extension
beyond two stand-ins the loader registers.  This recipe copies the `pace/` package
directory of a reference checkout, as it lies, into `oracle/_ref/pace/` - a directory
that is ignored by git (nothing of the reference enters the history) but travels with
the working tree to a GPU box, where `bench.py --impl reference` and the `cpu_baseline`
leg then time the reference's own classes on the host cores (`kind: "reference"`).
Without the staged copy those legs time the restatement in oracle/cpu_path.py
(`kind: "port"`).

The reference root is the argument, else $PACE_REF_ROOT, else a `reference/` directory
beside this repository.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def default_root() -> str:
    env = os.environ.get("PACE_REF_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def stage(root: str = "") -> str:
    """Copies <root>/pace (Python files only) to oracle/_ref/pace; returns the destination or ""."""
    root = root or default_root()
    src = os.path.join(root, "pace")
    if not os.path.isfile(os.path.join(src, "llm", "cache.py")):
        return ""
    dst = os.path.join(DEST, "pace")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=lambda d, names: [n for n in names
                                                        if n == "__pycache__" or (os.path.isfile(os.path.join(d, n))
                                                                                  and not n.endswith(".py"))])
    with open(os.path.join(DEST, "STAGED_FROM"), "w") as f:
        f.write("the reference's pace/ package, copied unmodified by oracle/stage_ref.py\n")
    return dst


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else "")
    print(out or "no reference checkout found: nothing staged")
