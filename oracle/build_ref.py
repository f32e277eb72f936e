"""Recipe for oracle/_ref/: puts the reference's validation module where oracle/ref_runner.py
loads it from.

    python oracle/build_ref.py [/path/to/reference]

Without an argument the checkout is looked for in $RAPTOR_T_REFERENCE and then in a directory named
`reference` beside this repository.

The reference's path is Python, so "building" it is taking python/modeling_big_bird.py as it
lies in the checkout; nothing is edited.  oracle/_ref/ is git-ignored: the file never enters
this repository's history, it only travels next to the built libraries to the machine that
runs the benchmark.  Without a checkout this is a no-op and the CPU baseline falls back to the
restatement in oracle/bigbird.py.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _default_root():
    env = os.environ.get("RAPTOR_T_REFERENCE")
    if env:
        return env
    return os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def build(ref_root=None):
    src = os.path.join(ref_root or _default_root(), "python", "modeling_big_bird.py")
    dst_dir = os.path.join(HERE, "_ref")
    if not os.path.exists(src):
        return None
    os.makedirs(dst_dir, exist_ok=True)
    dst = os.path.join(dst_dir, "modeling_big_bird.py")
    shutil.copyfile(src, dst)
    return dst


if __name__ == "__main__":
    print(build(*sys.argv[1:2]) or "no reference checkout: nothing to do")
