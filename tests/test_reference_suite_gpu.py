"""The drop-in proof: the reference project's OWN test files, unmodified, run against this package
under the name `flag_attn`.

The files (tests/flag_attn/test_{flash,piecewise,paged}_attention.py and test_dropout.py of
FlagOpen/FlagAttention) are not part of this repository.  They are looked for in the directory named
by the environment variable FLAG_ATTN_REFERENCE_TESTS, else in baseline/_ref/tests/flag_attn (where
tests/stage_reference_tests.py puts them); without them the tests are skipped.  Each file is loaded
by path; for every test function in it, the full cartesian product of its own `parametrize` marks
is enumerated and a seeded sample of it is called as is (FLAG_ATTN_REFERENCE_CASES per function,
default 8: the full products run to thousands of cases).  `import flag_attn` inside those files
resolves to the alias package at the root of this repository.
"""
import importlib.util
import itertools
import os
import random
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FILES = ["test_flash_attention.py", "test_piecewise_attention.py", "test_paged_attention.py",
         "test_dropout.py"]


def _suite_dir():
    d = os.environ.get("FLAG_ATTN_REFERENCE_TESTS")
    if d and os.path.isdir(d):
        return d
    d = os.path.join(ROOT, "baseline", "_ref", "tests", "flag_attn")
    return d if os.path.isdir(d) else None


def _cases(fn):
    """Every parameter combination pytest would generate for `fn`, as keyword dictionaries."""
    axes = []
    for mark in getattr(fn, "pytestmark", []):
        if mark.name != "parametrize":
            continue
        names, values = mark.args[0], mark.args[1]
        if isinstance(names, str):
            names = [n.strip() for n in names.split(",")]
        rows = []
        for v in values:
            v = getattr(v, "values", v)          # pytest.param(...)
            rows.append(dict(zip(names, v if len(names) > 1 else [v])))
        axes.append(rows)
    out = []
    for combo in itertools.product(*axes):
        kw = {}
        for part in combo:
            kw.update(part)
        out.append(kw)
    return out


@pytest.mark.parametrize("filename", FILES)
def test_reference_test_file_passes_unmodified(filename):
    suite = _suite_dir()
    if suite is None or not os.path.exists(os.path.join(suite, filename)):
        pytest.skip("the reference's test files are not staged on this machine")
    import flag_attn
    assert os.path.dirname(os.path.dirname(os.path.abspath(flag_attn.__file__))) == ROOT, \
        "flag_attn must resolve to this repository's package"
    spec = importlib.util.spec_from_file_location("reference_suite_" + filename[:-3],
                                                  os.path.join(suite, filename))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    per_fn = int(os.environ.get("FLAG_ATTN_REFERENCE_CASES", "8"))
    ran = 0
    for name in sorted(n for n in dir(mod) if n.startswith("test_") and callable(getattr(mod, n))):
        fn = getattr(mod, name)
        cases = _cases(fn)
        assert cases, f"{filename}::{name} has no cases (no CUDA device?)"
        rng = random.Random(10086 + len(cases))
        for kw in (rng.sample(cases, per_fn) if len(cases) > per_fn else cases):
            try:
                fn(**kw)
            except AssertionError as e:
                raise AssertionError(f"{filename}::{name}{kw}: {e}") from e
            finally:
                # the paged file switches torch's process-wide defaults (fp16, "cuda") and never
                # switches them back; the tests that follow in this process must not inherit that
                torch.set_default_dtype(torch.float32)
                torch.set_default_device("cpu")
            ran += 1
            torch.cuda.empty_cache()
    assert ran > 0
    print(f"{filename}: {ran} cases of the reference's own tests passed", file=sys.stderr)
