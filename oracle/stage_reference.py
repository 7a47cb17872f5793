"""Stages the reference package (pure Python) under oracle/_ref/ so that it can travel to the GPU box.

    python oracle/stage_reference.py [/path/to/reference]

The reference has nothing to compile: "building" it is installing its `stk` package directory.  The
copy lands in oracle/_ref/stk (git-ignored: it never enters the history), without the reference's
test files.  TEST / BASELINE INFRASTRUCTURE ONLY: bench.py's `--impl reference` and `cpu_baseline`
legs and `python -m stk_b200.benchmarks ref` import it from there; nothing in stk_b200/ does.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")


def stage(source="/root/reference"):
    """Returns the staged package path, or None when the reference is not present here."""
    pkg = os.path.join(source, "stk")
    if not os.path.isdir(pkg):
        return None
    dest = os.path.join(TARGET, "stk")
    if os.path.isdir(dest):
        shutil.rmtree(dest)
    os.makedirs(TARGET, exist_ok=True)
    shutil.copytree(pkg, dest, ignore=shutil.ignore_patterns("*_test.py", "__pycache__"))
    return dest


def import_reference():
    """The staged reference as a module (`import stk` resolved to oracle/_ref/stk), or None."""
    if not os.path.isdir(os.path.join(TARGET, "stk")):
        return None
    if TARGET not in sys.path:
        sys.path.insert(0, TARGET)
    import stk  # noqa: E402 - the reference package
    return stk


if __name__ == "__main__":
    print(stage(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))
