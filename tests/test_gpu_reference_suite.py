"""The reference project's own tests, unmodified, driven through the import-name shims.

Set SMLA_REFERENCE_TESTS to the root of a checkout of the reference (the folder that holds its
``tests/``); the run then imports ``flash_mla_sm120`` from THIS repository (the shim packages at
the repository root come first on PYTHONPATH) and executes the reference's test files in a child
pytest.  Without the variable the test is skipped: the reference is not part of this repository.
Every correctness test file of the reference is run whole (both cache layouts, the second cache, sink,
lengths, CUDA-graph capture, NaN safety, padded strides); its perf and profiling scripts are not.
"""
import os
import subprocess
import sys

import pytest

from helpers import ROOT

pytestmark = pytest.mark.gpu

# file -> pytest -k expression ("" = the whole file)
SELECTION = {
    "tests/test_decode.py": "",
    "tests/test_decode_v2.py": "",
    "tests/test_prefill.py": "",
    "tests/test_combine.py": "",
    "tests/test_scheduler.py": "",
    "tests/test_nan_safe.py": "",
    "tests/test_precision_magnitude.py": "",
    "tests/test_v4_features.py": "",
}


@pytest.mark.parametrize("path", sorted(SELECTION))
def test_reference_file(path):
    ref = os.environ.get("SMLA_REFERENCE_TESTS")
    if not ref or not os.path.exists(os.path.join(ref, path)):
        pytest.skip("SMLA_REFERENCE_TESTS does not point at a checkout of the reference")
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "pytest", path, "-q", "-rf", "--tb=line", "-p", "no:cacheprovider"]
    if SELECTION[path]:
        cmd += ["-k", SELECTION[path]]
    res = subprocess.run(cmd, cwd=ref, env=env, capture_output=True, text=True, timeout=1200)
    tail = (res.stdout + res.stderr)[-6000:]
    log = os.environ.get("SMLA_REFERENCE_LOG")
    if log:
        with open(log, "a") as f:
            f.write(f"==== {path} -k '{SELECTION[path]}' -> rc {res.returncode}\n{tail}\n")
    assert res.returncode == 0, tail
