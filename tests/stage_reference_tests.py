"""Stages the reference project's own test files where test_reference_suite_gpu.py looks for them.

    python tests/stage_reference_tests.py <path of a FlagOpen/FlagAttention checkout>

copies <checkout>/tests/flag_attn/test_*.py, unmodified, into baseline/_ref/tests/flag_attn/ at the
root of this repository.  That folder is ignored by git (the files are the reference's, not this
project's) but it travels with the working tree to the machine that runs the GPU tests, which has
no checkout of the reference.
"""
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEST = os.path.join(ROOT, "baseline", "_ref", "tests", "flag_attn")


def main(checkout):
    src = os.path.join(checkout, "tests", "flag_attn")
    names = sorted(n for n in os.listdir(src) if n.startswith("test_") and n.endswith(".py"))
    if not names:
        raise SystemExit("no test files under %s" % src)
    os.makedirs(DEST, exist_ok=True)
    for n in names:
        shutil.copyfile(os.path.join(src, n), os.path.join(DEST, n))
    print("staged %d files in %s" % (len(names), DEST))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
