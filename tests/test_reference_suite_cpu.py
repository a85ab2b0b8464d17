"""The reference's own python tests for the buffer, batching and slicing API,
run unmodified against this package.

The files are executed where they lie in the reference's source tree
(REFERENCE_ROOT, else a checkout named "reference" beside this repository);
none of their text is in this repository.  Without the tree the tests skip -
tests/test_stream_batching_cpu.py checks the same behaviour against the
compiled reference or by properties.  The samples in these files are plain
host arrays, so no GPU is needed.
"""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_ROOT = os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")

# file -> number of tests it holds that must run and pass
FILES = {"test_buffer.py": 4, "test_dynamic_batch.py": 6, "test_general_ops.py": 2}


@pytest.mark.parametrize("name", sorted(FILES))
def test_reference_file_passes(name):
    path = os.path.join(REFERENCE_ROOT, "python", "tests", name)
    if not os.path.isfile(path):
        pytest.skip("no reference tree (set REFERENCE_ROOT)")
    run = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "run_reference_tests.py"), path],
                         capture_output=True, text=True, timeout=600)
    tail = (run.stdout + run.stderr)[-4000:]
    assert run.returncode == 0, tail
    m = re.search(r"REFERENCE-TESTS ran=(\d+) failed=(\d+)", run.stdout)
    assert m, tail
    assert int(m.group(1)) >= FILES[name] and int(m.group(2)) == 0, tail
